"""CPU tests: the oracle against the reference's own code and golden vectors, the host-side layout logic, the C ABI's
exports, and the expert-parallel sharding rule over a 2-rank gloo group.  None of these needs a GPU."""
import ctypes as C
import pathlib
import re
import subprocess
import sys

import numpy as np
import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]
GOLD = ROOT / "tests" / "golden"


@pytest.fixture(scope="module")
def pins():
    return np.load(GOLD / "ref_pins.npz")


@pytest.fixture(scope="module")
def cases():
    return np.load(GOLD / "oracle_cases.npz")


def vp(a):
    return a.ctypes.data_as(C.c_void_p)


# ------------------------------------------------------------------------------------------------ pins against the reference
def test_grid_equals_reference_and_gguf(O, pins):
    g = O.grid()
    assert np.array_equal(g, pins["iq3s_grid"])
    from gguf.quants import IQ3_S
    IQ3_S.init_grid()
    gg = np.asarray(IQ3_S.grid).reshape(512, 4).astype(np.uint32)
    assert np.array_equal(g, gg[:, 0] | gg[:, 1] << 8 | gg[:, 2] << 16 | gg[:, 3] << 24)


def test_dequant_bit_equal_to_reference_vectors(O, pins):
    got = O.iq3s_dequant(pins["iq3s_blocks"])
    assert np.array_equal(got.view(np.uint32), pins["iq3s_values"].view(np.uint32))


def test_dequant_bit_equal_to_gguf_py(O):
    from gguf import GGMLQuantizationType as QT
    from gguf.quants import dequantize
    rng = np.random.default_rng(7)
    blk = rng.integers(0, 256, size=(500, 110), dtype=np.uint8)
    d = blk[:, :2].view(np.uint16)
    d[(d & 0x7C00) == 0x7C00] &= 0x3FFF
    assert np.array_equal(O.iq3s_dequant(blk).view(np.uint32), dequantize(blk, QT.IQ3_S).reshape(500, 256).view(np.uint32))


def test_live_reference_build_when_present(O):
    r = O.ref()
    if r is None:
        pytest.skip("oracle/_ref not built here (no reference checkout)")
    rng = np.random.default_rng(8)
    blk = rng.integers(0, 256, size=(300, 110), dtype=np.uint8)
    d = blk[:, :2].view(np.uint16)
    d[(d & 0x7C00) == 0x7C00] &= 0x3FFF
    out = np.empty((300, 256), np.float32)
    r.ref_iq3s_dequant(vp(blk), C.c_size_t(300), vp(out))
    assert np.array_equal(O.iq3s_dequant(blk).view(np.uint32), out.view(np.uint32))
    for x in (rng.standard_normal(300) * 10.0 ** rng.integers(-8, 5, 300)).astype(np.float32):
        assert O.lib().fnx_o_f2h(C.c_float(float(x))) == r.ref_f2h(C.c_float(float(x)))


def test_f2h_matches_reference_vectors(O, pins):
    got = np.array([O.lib().fnx_o_f2h(C.c_float(float(x))) for x in pins["f2h_in"]], np.uint16)
    assert np.array_equal(got, pins["f2h_out"])


def test_make_dist_and_draw_match_reference_vectors(O, pins):
    for i in range(len(pins["md_n"])):
        t, tp, mp, tk = pins["md_par"][i]
        s = O.Sampling(float(t), float(tp), float(mp), int(tk))
        ids, p = O.make_dist(pins["md_v"][i], pins["md_i"][i], s)
        n = int(pins["md_n"][i])
        assert len(ids) == n and np.array_equal(ids, pins["md_ids"][i][:n])
        assert np.array_equal(p, pins["md_p"][i][:n])          # same doubles, bit for bit
        assert O.draw(ids, p, float(pins["md_u"][i])) == int(pins["md_pick"][i])


def test_lookup_matches_reference_vectors(O, pins):
    ctx = pins["lk_ctx"]
    hits = 0
    for row in pins["lk_cases"]:
        n, lk, d1, cnt, m = (int(v) for v in row[:5])
        out, match = O.lookup(ctx[:n], lk, d1)
        assert len(out) == cnt and match == m and list(out) == [int(v) for v in row[5:5 + cnt]]
        hits += cnt > 0
    assert hits > 20


def test_philox_known_answers(O):
    # Random123's published known-answer vectors for philox4x32-10
    assert list(O.philox([0, 0, 0, 0], [0, 0])) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert list(O.philox([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2)) == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    assert list(O.philox([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0])) == [0xD16CFE09, 0x94FDCCEB, 0x5001E420,
                                                                                                        0x24126EA1]
    u = [O.uniform(5, 1, 2, s) for s in range(1000)]
    assert 0.0 <= min(u) and max(u) < 1.0 and abs(np.mean(u) - 0.5) < 0.05


# ------------------------------------------------------------------------------------------------ oracle golden cases
def test_oracle_reproduces_golden_cases(O, cases):
    c = cases
    out, logits, topi, topw = O.moe(c["moe_wr"], c["moe_wgu"], c["moe_wdn"], c["moe_sgu"], c["moe_sdn"], c["moe_x"], 256, 2)
    assert np.array_equal(topi, c["moe_topi"]) and np.array_equal(out, c["moe_out"]) and np.array_equal(topw, c["moe_topw"])
    qg, k, kc, vc = c["at_qg_in"].copy(), c["at_k_in"].copy(), c["at_kc_in"].copy(), c["at_vc_in"].copy()
    O.attn_prep_append(qg, k, c["at_v"], c["at_qn"], c["at_kn"], kc, vc, int(c["at_pos0"]), c["at_depth"], 64)
    assert np.array_equal(qg, c["at_qg"]) and np.array_equal(kc, c["at_kc"]) and np.array_equal(vc, c["at_vc"])
    assert np.array_equal(O.attn(qg, kc, vc, int(c["at_pos0"]), c["at_parent"]), c["at_out"])
    sys.path.insert(0, str(GOLD))
    from make_golden import gdn_start_state
    S = gdn_start_state(5, 2, 128)
    hist = c["gd_hist_in"].copy()
    y = O.gdn_core(c["gd_qkvz"], c["gd_ab"], hist, c["gd_convw"], c["gd_dt"], c["gd_a"], c["gd_nw"], S, 2, c["gd_parent"], 1, 2, 128)
    assert np.array_equal(y, c["gd_y"]) and np.array_equal(hist, c["gd_hist"])
    assert np.array_equal(S.astype(np.float64).sum(axis=-1), c["gd_S_rowsum"])


def test_router_semantics(O):
    rng = np.random.default_rng(3)
    E, H, K, T = 64, 512, 10, 6
    wr = (rng.standard_normal((E + 1, H)) * 0.02).astype(np.float32)
    x = rng.standard_normal((T, H)).astype(np.float32)
    logits, topi, topw = O.router(wr, x, K)
    ref = (x.astype(np.float64) @ wr.astype(np.float64).T).astype(np.float32)
    assert np.array_equal(logits, ref)
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-ref[t, e], e))[:K]
        assert list(topi[t]) == order
        w = np.exp(ref[t, order].astype(np.float64) - ref[t, order[0]])
        assert np.allclose(topw[t], w / w.sum(), rtol=1e-6)
    # ties go to the lower index
    wr[5] = wr[9]
    _, topi, _ = O.router(wr, x, K)
    for t in range(T):
        li = list(topi[t])
        if 9 in li:
            assert 5 in li and li.index(5) < li.index(9)


def test_gdn_chain_equals_parent_minus_one_tree_and_delta_rule(O):
    rng = np.random.default_rng(5)
    nk, nv, hs, T, NS = 1, 2, 128, 3, 4
    ch = (2 * nk + nv) * hs
    qkvz = rng.standard_normal((T, ch + nv * hs)).astype(np.float32)
    ab = rng.standard_normal((T, 2 * nv)).astype(np.float32)
    convw = (0.5 * rng.standard_normal((ch, 4))).astype(np.float32)
    dt, a, nw = np.zeros(nv, np.float32), -np.ones(nv, np.float32), np.ones(hs, np.float32)
    S1 = (0.1 * rng.standard_normal((NS, nv, hs, hs))).astype(np.float32)
    h1 = rng.standard_normal((NS, 3, ch)).astype(np.float32)
    S2, h2 = S1.copy(), h1.copy()
    y1 = O.gdn_core(qkvz, ab, h1, convw, dt, a, nw, S1, 1, None, nk, nv, hs)
    y2 = O.gdn_core(qkvz, ab, h2, convw, dt, a, nw, S2, 1, [-1, 0, 1], nk, nv, hs)
    assert np.array_equal(y1, y2) and np.array_equal(S1, S2) and np.array_equal(h1, h2)
    # two siblings of the root see the same starting state: a window of one row gives each its own result
    S3, h3 = S1.copy(), h1.copy()
    y3 = O.gdn_core(qkvz[[0, 1, 2]], ab[[0, 1, 2]], h3, convw, dt, a, nw, S3, 1, [-1, 0, 0], nk, nv, hs)
    S4, h4 = S1.copy(), h1.copy()
    y4 = O.gdn_core(qkvz[[0, 2]], ab[[0, 2]], h4, convw, dt, a, nw, S4, 1, [-1, 0], nk, nv, hs)
    assert np.array_equal(y3[2], y4[1]) and np.array_equal(S3[(1 + 1 + 2) % NS], S4[(1 + 1 + 1) % NS])


def test_accept_rules(O):
    # greedy chain: accept while the draft equals the previous row's argmax (session.cpp:573)
    assert O.accept_greedy([5, 1, 2, 3], None, [1, 2, 9, 4])[0] == 3
    n, path, em = O.accept_greedy([5, 7, 1, 2, 8], [-1, 0, 0, 2, 2], [1, 0, 2, 0, 0])
    assert (n, list(path), list(em)) == (3, [0, 2, 3], [1, 2, 0])
    # sampling: a draft the target gives probability ~1 always stands; one it gives 0 never does
    cv = np.full((2, 64), -30.0, np.float32)
    cv[:, 0] = 10.0
    ci = np.tile(np.arange(64, dtype=np.int32), (2, 1))
    s = O.Sampling(1.0, 1.0, 0.0, 0)
    for step in range(20):
        assert O.accept_sample(cv, ci, [3, 0], s, 9, 0, step)[0] == 2
        n, em = O.accept_sample(cv, ci, [3, 63], s, 9, 0, step)
        assert n == 1 and em[0] != 63


# ------------------------------------------------------------------------------------------------ host-side layout logic
@pytest.fixture(scope="module")
def sim(tmp_path_factory):
    out = tmp_path_factory.mktemp("sim") / "libtile_sim.so"
    pk = ROOT / "qwen3.8-flash-next-2x-p100_b200" / "csrc"
    subprocess.run(["/usr/bin/g++" if pathlib.Path("/usr/bin/g++").exists() else "g++", "-O2", "-std=c++17", "-shared", "-fPIC", f"-I{pk}", "-o",
                    str(out), str(ROOT / "tests" / "csrc" / "tile_sim.cpp")], check=True)
    return C.CDLL(str(out))


def test_tile_layout_round_trip_and_warp_replay(O, sim):
    rng = np.random.default_rng(1)
    for rows, K, T in [(16, 256, 1), (64, 1024, 3), (32, 2048, 4)]:
        blk = rng.integers(0, 256, size=(rows * (K // 256), 110), dtype=np.uint8)
        back = np.empty_like(blk)
        sim.sim_roundtrip(vp(blk), rows, K, vp(back))
        assert np.array_equal(blk, back)
        q = O.iq3s_quantize((rng.standard_normal((rows, K)) * 0.02).astype(np.float32))
        x = rng.standard_normal((T, K)).astype(np.float32)
        y = np.zeros((T, rows), np.float32)
        sim.sim_mmv(vp(q), rows, K, vp(x), T, vp(y))
        ref = O.iq3s_gemv(q, rows, K, x)
        assert np.abs(y - ref).max() <= 2e-4 * np.abs(ref).max()


def test_c_abi_exports_every_declared_symbol(F):
    hdr = (ROOT / "include" / "fnx_b200.h").read_text()
    declared = set(re.findall(r"\b(fnx_[a-z0-9_]+)\s*\(", hdr))
    assert declared == set(F.EXPORTS)
    L = F.lib()
    for name in declared:
        assert hasattr(L, name), name
    assert L.fnx_version() >= 100
    assert L.fnx_iq3s_bytes(16, 256) == 1760 and F.iq3s_bytes(2048, 512) == 450560


def test_header_is_plain_c(tmp_path):
    """The header is what a cgo / ctypes / JNI binding includes: it has to compile as C, not only as C++."""
    import shutil
    import subprocess
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "includes_header.c"
    src.write_text('#include "fnx_b200.h"\nint main(void) { return fnx_iq3s_bytes(16, 256) == 1760 ? 0 : 1; }\n')
    r = subprocess.run([cc, "-std=c11", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", f"-I{ROOT / 'include'}", str(src)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_engine_argument_checks_need_no_gpu(F):
    L = F.lib()
    assert L.fnx_dense(None, 64, 2048, None, 2048, 1, None, 1e-6, None, 64, 0, None, None) == -1
    assert b"null" in L.fnx_last_error()
    assert L.fnx_dense(None, 64, 700, None, 700, 1, None, 1e-6, None, 64, 0, None, None) == -1
    assert L.fnx_iq3s_retile(None, None, 10, 256, None) == -1


# ------------------------------------------------------------------------------------------------ the lane planner (host arithmetic)
def test_lane_planner_finds_the_best_rate(F):
    """fnx_plan_rows against an exhaustive search over every draft count: the plan's expected tokens per ms is the maximum
    (costs with a knee inside the window, chain lanes whose later drafts cost a call each, a row budget that binds)."""
    import itertools
    rng = np.random.default_rng(4)
    for case in range(40):
        n = int(rng.integers(1, 5))
        avail = [int(rng.integers(0, 5)) for _ in range(n)]
        reach = [np.sort(rng.uniform(0.05, 0.95, size=4))[::-1].tolist() for _ in range(n)]
        chain = [bool(rng.integers(0, 2)) for _ in range(n)]
        max_rows = int(rng.integers(n, min(32, n + 9) + 1))
        base, lo, hi, ch, knee = float(rng.uniform(2, 12)), float(rng.uniform(0.1, 1.5)), float(rng.uniform(1.5, 3.0)), float(rng.uniform(0.0, 0.8)), int(rng.integers(2, 12))

        def rate(d):
            tok, ms, rows = float(n), base, n
            for i in range(n):
                tok += sum(reach[i][:d[i]])
                ms += max(0, d[i] - 1) * ch if chain[i] else 0.0
            for t in range(n + 1, n + sum(d) + 1):
                ms += lo if t <= knee else hi
            return tok / ms

        best = max(rate(d) for d in itertools.product(*[range(min(a, 4) + 1) for a in avail]) if sum(d) <= max_rows - n)
        d, r = F.plan_rows(avail, reach, chain, max_rows, base, lo, hi, ch, knee)
        assert all(0 <= d[i] <= min(avail[i], 4) for i in range(n)) and sum(d) <= max_rows - n
        assert abs(rate(d) - best) <= 1e-12 * best and abs(r - best) <= 1e-9 * best, (case, d, rate(d), best)


# ------------------------------------------------------------------------------------------------ expert-parallel rule, 2 ranks on gloo
_EP_WORKER = r"""
import sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[3])
import oracle as O
rank, world = int(sys.argv[1]), 2
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{sys.argv[2]}", rank=rank, world_size=world)
c = np.load(sys.argv[3] + "/tests/golden/oracle_cases.npz")
E = c["moe_wr"].shape[0] - 1
lo, hi = rank * E // world, (rank + 1) * E // world
part, _, topi, _ = O.moe(c["moe_wr"], c["moe_wgu"], c["moe_wdn"], c["moe_sgu"], c["moe_sdn"], c["moe_x"], 256, 2, e_lo=lo, e_hi=hi, add_shared=False)
t = torch.from_numpy(part.astype(np.float64))
dist.all_reduce(t)
shared, _, _, _ = O.moe(c["moe_wr"], c["moe_wgu"], c["moe_wdn"], c["moe_sgu"], c["moe_sdn"], c["moe_x"], 256, 2, e_lo=0, e_hi=0, add_shared=True)
total = t.numpy() + shared
assert np.array_equal(topi, c["moe_topi"])
err = np.abs(total - c["moe_out"]).max() / np.abs(c["moe_out"]).max()
assert err < 1e-6, err
dist.destroy_process_group()
print("ok", rank)
"""


def test_expert_parallel_partial_sums_two_ranks_gloo(tmp_path):
    script = tmp_path / "ep_worker.py"
    script.write_text(_EP_WORKER)
    port = 29500 + (abs(hash(str(tmp_path))) % 2000)
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(port), str(ROOT)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o


# ------------------------------------------------------------------------------------------------ sequence-sharded mixers, 2 ranks on gloo
_DP_WORKER = r"""
import sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[3])
import oracle as O
rank, world = int(sys.argv[1]), 2
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{sys.argv[2]}", rank=rank, world_size=world)
# a lanes window of 3 sequences x 2 rows: every rank has every row's queries, but the caches of its own sequences only
rng = np.random.default_rng(7)
nq, nkv, hd, rows, seqs = 4, 1, 256, 2, [0, 1, 2]
pos = {0: 5, 1: 9, 2: 3}
qg = rng.standard_normal((len(seqs) * rows, nq, 2 * hd)).astype(np.float32)
caches = {s: ((rng.standard_normal((pos[s] + rows, nkv, hd))).astype(np.float16).view(np.uint16),
              (rng.standard_normal((pos[s] + rows, nkv, hd))).astype(np.float16).view(np.uint16)) for s in seqs}
full = np.concatenate([O.attn(qg[j * rows:(j + 1) * rows], caches[s][0], caches[s][1], pos[s], None) for j, s in enumerate(seqs)])
# the rule of the engine's lanes windows: lane j runs on rank seq % world; the others' rows are gathered
mine = np.zeros_like(full)
own = [s % world == rank for s in seqs]
for j, s in enumerate(seqs):
    if own[j]:
        mine[j * rows:(j + 1) * rows] = O.attn(qg[j * rows:(j + 1) * rows], caches[s][0], caches[s][1], pos[s], None)
t = torch.from_numpy(mine.copy())
dist.all_reduce(t)          # disjoint rows: the sum is the gather
assert sum(own) in (1, 2) and np.array_equal(t.numpy(), full)
dist.destroy_process_group()
print("ok", rank)
"""


def test_sequence_sharded_mixers_two_ranks_gloo(tmp_path):
    """Lanes windows on expert-parallel ranks: each rank computes the attention of its own sequences' lanes (sequence % ranks
    == rank) and the rows are gathered: the gathered rows equal the single-rank result bit for bit."""
    script = tmp_path / "dp_worker.py"
    script.write_text(_DP_WORKER)
    port = 31500 + (abs(hash(str(tmp_path))) % 2000)
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(port), str(ROOT)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o
