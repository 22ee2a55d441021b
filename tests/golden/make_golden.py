"""Generates the committed golden fixtures; needs a checkout of the reference (oracle/Makefile's REF) for ref_pins.npz.

    python tests/golden/make_golden.py

ref_pins.npz    outputs of the REFERENCE's own host code (oracle/_ref: engine/src/tensor_convert.hpp dequantize,
                engine/src/session.cpp make_dist / draw / lookup_drafts) on seeded inputs: the vectors carry the
                pins to machines without a reference checkout.
oracle_cases.npz  small seeded operator cases with the oracle's outputs: they pin the oracle against accidental
                change and give the GPU tests fixed inputs.
"""
import ctypes as C
import pathlib
import sys

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import oracle as O  # noqa: E402

OUT = pathlib.Path(__file__).resolve().parent


def vp(a):
    return a.ctypes.data_as(C.c_void_p)


def ref_pins():
    O.build(ref=True)
    r = O.ref()
    assert r is not None, "the reference pins need a reference checkout (oracle/Makefile: REF)"
    rng = np.random.default_rng(100)
    d = {}
    blk = rng.integers(0, 256, size=(64, 110), dtype=np.uint8)
    dd = blk[:, :2].view(np.uint16)
    dd[(dd & 0x7C00) == 0x7C00] &= 0x3FFF
    out = np.empty((64, 256), np.float32)
    r.ref_iq3s_dequant(vp(blk), C.c_size_t(64), vp(out))
    d["iq3s_blocks"], d["iq3s_values"] = blk, out
    d["iq3s_grid"] = np.ctypeslib.as_array(r.ref_iq3s_grid(), shape=(512,)).copy()
    fl = np.concatenate([rng.standard_normal(200).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1.0, 100.0, 7e4)])
    d["f2h_in"] = fl
    d["f2h_out"] = np.array([r.ref_f2h(C.c_float(float(x))) for x in fl], np.uint16)
    # make_dist / draw
    cv, ci, par, ids, ps, ns, us, picks = [], [], [], [], [], [], [], []
    for i in range(40):
        v = np.sort((rng.standard_normal(64) * 3).astype(np.float32))[::-1].copy()
        idx = rng.permutation(5000)[:64].astype(np.int32)
        t, tp, mp, tk = [(0.7, 1.0, 0.0, 0), (1.0, 0.9, 0.0, 0), (0.5, 1.0, 0.05, 0), (1.3, 0.95, 0.02, 20)][i % 4]
        oi = np.zeros(64, np.int32)
        op = np.zeros(64, np.float64)
        n = r.ref_make_dist(vp(v), vp(idx), 64, t, tp, mp, tk, vp(oi), vp(op))
        u = float(rng.random())
        pick = r.ref_draw(vp(oi), vp(op), n, C.c_double(u))
        cv.append(v); ci.append(idx); par.append([t, tp, mp, tk]); ids.append(oi); ps.append(op); ns.append(n); us.append(u); picks.append(pick)
    d.update(md_v=np.array(cv), md_i=np.array(ci), md_par=np.array(par, np.float64), md_ids=np.array(ids), md_p=np.array(ps),
             md_n=np.array(ns, np.int32), md_u=np.array(us), md_pick=np.array(picks, np.int32))
    # lookup_drafts
    ctx = rng.integers(0, 50, size=4000).astype(np.int32)
    ctx[2000:2300] = ctx[500:800]
    ctx[3500:3600] = ctx[2100:2200]
    cases = []
    for n in list(rng.integers(4, 4000, size=150)) + [2, 3, 4, 2300, 3600, 4000]:
        for lk in (15, 4, 0):
            for d1 in (-1, int(ctx[min(int(n), 3999)]), 49):
                out_t = np.full(16, -1, np.int32)
                m = C.c_int(-9)
                cnt = r.ref_lookup(vp(ctx), int(n), lk, d1, vp(out_t), C.byref(m))
                cases.append([int(n), lk, d1, cnt, m.value] + out_t[:15].tolist())
    d["lk_ctx"], d["lk_cases"] = ctx, np.array(cases, np.int32)
    np.savez_compressed(OUT / "ref_pins.npz", **d)
    print("ref_pins.npz", (OUT / "ref_pins.npz").stat().st_size)


def gdn_start_state(NS, nv, hs):
    i = np.arange(NS * nv * hs * hs, dtype=np.float64)
    return (0.1 * np.sin(0.37 * i + 0.11 * (i % 97))).astype(np.float32).reshape(NS, nv, hs, hs)


def oracle_cases():
    rng = np.random.default_rng(200)
    d = {}
    # a small MoE block: 8 experts, hidden 256, ffn 256, top 2, 3 rows
    E, H, Fn, K, T = 8, 256, 256, 2, 3
    wr = (rng.standard_normal((E + 1, H)) * 0.02).astype(np.float32)
    wgu = O.iq3s_quantize((rng.standard_normal((E, 2 * Fn, H)) * 0.02).astype(np.float32)).reshape(-1)
    wdn = O.iq3s_quantize((rng.standard_normal((E, H, Fn)) * 0.02).astype(np.float32)).reshape(-1)
    sgu = O.iq3s_quantize((rng.standard_normal((2 * Fn, H)) * 0.02).astype(np.float32)).reshape(-1)
    sdn = O.iq3s_quantize((rng.standard_normal((H, Fn)) * 0.02).astype(np.float32)).reshape(-1)
    x = rng.standard_normal((T, H)).astype(np.float32)
    out, logits, topi, topw = O.moe(wr, wgu, wdn, sgu, sdn, x, Fn, K)
    d.update(moe_wr=wr, moe_wgu=wgu, moe_wdn=wdn, moe_sgu=sgu, moe_sdn=sdn, moe_x=x, moe_out=out, moe_logits=logits, moe_topi=topi, moe_topw=topw)
    # attention: 2 q heads per KV head would be unusual; keep the model's 8
    nq, nkv, hd, pos0, T = 8, 1, 256, 21, 4
    kc = np.zeros((pos0 + T, nkv, hd), np.uint16)
    vc = np.zeros((pos0 + T, nkv, hd), np.uint16)
    kc[:pos0] = rng.standard_normal((pos0, nkv, hd)).astype(np.float16).view(np.uint16)
    vc[:pos0] = rng.standard_normal((pos0, nkv, hd)).astype(np.float16).view(np.uint16)
    qg = rng.standard_normal((T, nq, 2 * hd)).astype(np.float32)
    k = rng.standard_normal((T, nkv, hd)).astype(np.float32)
    v = rng.standard_normal((T, nkv, hd)).astype(np.float32)
    qn = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    kn = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    parent = np.array([-1, 0, 0, 2], np.int32)
    depth = np.array([0, 1, 1, 2], np.int32)
    d.update(at_qg_in=qg.copy(), at_k_in=k.copy(), at_v=v, at_qn=qn, at_kn=kn, at_kc_in=kc.copy(), at_vc_in=vc.copy(), at_parent=parent,
             at_depth=depth, at_pos0=np.int32(pos0))
    O.attn_prep_append(qg, k, v, qn, kn, kc, vc, pos0, depth, 64)
    d.update(at_qg=qg, at_kc=kc, at_vc=vc, at_out=O.attn(qg, kc, vc, pos0, parent))
    # DeltaNet: 1 key head, 2 value heads, a 4-row tree; the starting state is a formula, not stored
    nk, nv, hs, T, NS = 1, 2, 128, 4, 5
    ch = (2 * nk + nv) * hs
    qkvz = rng.standard_normal((T, ch + nv * hs)).astype(np.float32)
    ab = rng.standard_normal((T, 2 * nv)).astype(np.float32)
    convw = (0.5 * rng.standard_normal((ch, 4))).astype(np.float32)
    dt = (0.1 * rng.standard_normal(nv)).astype(np.float32)
    a = (-np.exp(0.3 * rng.standard_normal(nv))).astype(np.float32)
    nw = (1 + 0.1 * rng.standard_normal(hs)).astype(np.float32)
    S = gdn_start_state(NS, nv, hs)
    hist = rng.standard_normal((NS, 3, ch)).astype(np.float32)
    d.update(gd_qkvz=qkvz, gd_ab=ab, gd_convw=convw, gd_dt=dt, gd_a=a, gd_nw=nw, gd_hist_in=hist.copy(), gd_parent=parent)
    y = O.gdn_core(qkvz, ab, hist, convw, dt, a, nw, S, 2, parent, nk, nv, hs)
    d.update(gd_y=y, gd_S_rowsum=S.astype(np.float64).sum(axis=-1), gd_hist=hist)
    np.savez_compressed(OUT / "oracle_cases.npz", **d)
    print("oracle_cases.npz", (OUT / "oracle_cases.npz").stat().st_size)


if __name__ == "__main__":
    ref_pins()
    oracle_cases()
