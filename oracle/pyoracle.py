"""ctypes/numpy front of the CPU oracle (test infrastructure only; see fnx_oracle.h)."""
from __future__ import annotations

import ctypes as C
import pathlib
import subprocess

import numpy as np

_HERE = pathlib.Path(__file__).resolve().parent
_LIB = None
_REF = None
TOPN = 64
BLOCK = 110


def build(ref: bool = True) -> None:
    """Compiles the restatement and, when a reference checkout is present, the reference pins."""
    subprocess.run(["make", "-C", str(_HERE)], check=True, capture_output=True)
    if ref:   # a no-op where the Makefile's REF checkout is absent
        subprocess.run(["make", "-C", str(_HERE), "ref"], check=True, capture_output=True)


def _p(a, t=None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(C.c_void_p)


class Sampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("min_p", C.c_float), ("top_k", C.c_int)]


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        so = _HERE / "_build" / "libfnx_oracle.so"
        if not so.exists():
            build(ref=False)
        _LIB = C.CDLL(str(so))
        _LIB.fnx_o_h2f.restype = C.c_float
        _LIB.fnx_o_h2f.argtypes = [C.c_uint16]
        _LIB.fnx_o_f2h.restype = C.c_uint16
        _LIB.fnx_o_f2h.argtypes = [C.c_float]
        _LIB.fnx_o_iq3s_grid.restype = C.POINTER(C.c_uint32)
        _LIB.fnx_o_uniform.restype = C.c_double
        _LIB.fnx_o_uniform.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32]
        _LIB.fnx_o_draw.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_double]
    return _LIB


def ref():
    """The reference's own host functions (None when oracle/_ref was not built)."""
    global _REF
    if _REF is None:
        so = _HERE / "_ref" / "libfnx_ref.so"
        if not so.exists():
            return None
        _REF = C.CDLL(str(so))
        _REF.ref_iq3s_grid.restype = C.POINTER(C.c_uint32)
        _REF.ref_f2h.restype = C.c_uint16
        _REF.ref_f2h.argtypes = [C.c_float]
        _REF.ref_h2f.restype = C.c_float
        _REF.ref_h2f.argtypes = [C.c_uint16]
        _REF.ref_draw.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_double]
        _REF.ref_make_dist.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_float, C.c_int,
                                       C.c_void_p, C.c_void_p]
    return _REF


def threads(n: int = 0) -> int:
    """Sets (n > 0) and returns the size of the oracle's OpenMP team."""
    return int(lib().fnx_o_threads(int(n)))


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def grid() -> np.ndarray:
    return np.ctypeslib.as_array(lib().fnx_o_iq3s_grid(), shape=(512,)).copy()


def iq3s_dequant(blocks: np.ndarray) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, BLOCK)
    out = np.empty((blocks.shape[0], 256), np.float32)
    lib().fnx_o_iq3s_dequant(_p(blocks), C.c_size_t(blocks.shape[0]), _p(out))
    return out


def iq3s_quantize(w: np.ndarray) -> np.ndarray:
    """float weights (last dim a multiple of 256) -> uint8 blocks [..., n/256 * 110]"""
    w = f32(w)
    n = w.size
    assert w.shape[-1] % 256 == 0
    out = np.empty(n // 256 * BLOCK, np.uint8)
    lib().fnx_o_iq3s_quantize(_p(w), C.c_size_t(n), _p(out))
    return out.reshape(w.shape[:-1] + (w.shape[-1] // 256 * BLOCK,))


def iq3s_gemv(W: np.ndarray, rows: int, cols: int, x: np.ndarray) -> np.ndarray:
    x = f32(x).reshape(-1, cols)
    W = np.ascontiguousarray(W, np.uint8)
    assert W.size == rows * (cols // 256) * BLOCK
    y = np.empty((x.shape[0], rows), np.float32)
    lib().fnx_o_iq3s_gemv(_p(W), rows, cols, _p(x), cols, x.shape[0], _p(y), rows)
    return y


def rmsnorm(x, w, eps=1e-6):
    x = f32(x)
    y = np.empty_like(x)
    lib().fnx_o_rmsnorm(_p(x), _p(f32(w)), _p(y), int(np.prod(x.shape[:-1])), x.shape[-1], C.c_float(eps))
    return y


def router(Wr, x, K=10):
    Wr, x = f32(Wr), f32(x)
    E, H, T = Wr.shape[0] - 1, Wr.shape[1], x.shape[0]
    logits = np.empty((T, E + 1), np.float32)
    topi = np.empty((T, K), np.int32)
    topw = np.empty((T, K), np.float32)
    lib().fnx_o_router(_p(Wr), _p(x), T, E, H, K, _p(logits), _p(topi), _p(topw))
    return logits, topi, topw


def moe(Wr, Wgu, Wdn, Wsh_gu, Wsh_dn, x, F, K=10, e_lo=0, e_hi=None, add_shared=True):
    Wr, x = f32(Wr), f32(x)
    E, H, T = Wr.shape[0] - 1, Wr.shape[1], x.shape[0]
    e_hi = E if e_hi is None else e_hi
    out = np.empty((T, H), np.float32)
    logits = np.empty((T, E + 1), np.float32)
    topi = np.empty((T, K), np.int32)
    topw = np.empty((T, K), np.float32)
    lib().fnx_o_moe(_p(Wr), _p(Wgu), _p(Wdn), _p(Wsh_gu), _p(Wsh_dn), _p(x), T, E, H, F, K, e_lo, e_hi,
                    1 if add_shared else 0, _p(out), _p(logits), _p(topi), _p(topw))
    return out, logits, topi, topw


def attn_prep_append(qg, k, v, qn, kn, kc, vc, pos0, depth=None, nrot=64, eps=1e-6, rope_base=1e7):
    """In place on qg [T][nq][2 hd], k [T][nkv][hd]; appends to kc / vc (uint16 [ctx][nkv][hd])."""
    T, nq, hd2 = qg.shape
    nkv, hd = k.shape[1], k.shape[2]
    d = None if depth is None else i32(depth)
    lib().fnx_o_attn_prep_append(_p(qg), _p(k), _p(f32(v)), _p(f32(qn)), _p(f32(kn)), _p(kc), _p(vc), T, nq, nkv, hd,
                                 int(nrot), int(pos0), _p(d), C.c_float(eps), C.c_float(rope_base))


def attn(qg, kc, vc, pos0, parent=None):
    T, nq, hd2 = qg.shape
    nkv, hd = kc.shape[1], kc.shape[2]
    out = np.empty((T, nq, hd), np.float32)
    par = None if parent is None else i32(parent)
    lib().fnx_o_attn(_p(qg), _p(kc), _p(vc), _p(out), T, nq, nkv, hd, int(pos0), _p(par))
    return out


def gdn_core(qkvz, ab, hist_pool, convw, dt, a, nw, S_pool, cur, parent, nk, nv, hs=128, eps=1e-6):
    """hist_pool [NS][3][ch] and S_pool [NS][nv][hs][hs] are updated in place; returns y [T][nv*hs]."""
    T = qkvz.shape[0]
    NS = S_pool.shape[0]
    y = np.empty((T, nv * hs), np.float32)
    par = None if parent is None else i32(parent)
    lib().fnx_o_gdn_core(_p(qkvz), _p(ab), _p(hist_pool), _p(f32(convw)), _p(f32(dt)), _p(f32(a)), _p(f32(nw)),
                         _p(S_pool), int(cur), int(NS), _p(par), _p(y), nk, nv, hs, T, C.c_float(eps))
    return y


def argmax(logits):
    logits = f32(logits)
    T, V = logits.shape
    bi = np.empty(T, np.int32)
    bv = np.empty(T, np.float32)
    lib().fnx_o_argmax(_p(logits), T, V, _p(bi), _p(bv))
    return bi, bv


def top_tokens(logits, n=TOPN):
    logits = f32(logits)
    T, V = logits.shape
    ov = np.empty((T, n), np.float32)
    oi = np.empty((T, n), np.int32)
    lib().fnx_o_top_tokens(_p(logits), T, V, n, _p(ov), _p(oi))
    return ov, oi


def logit_adjust(logits, ctx, tok, last_n=0, repeat=1.0, freq=0.0, present=0.0, bias=()):
    """The sampler's logit changes (bias list, then penalties over each row's window); returns a changed copy."""
    out = f32(logits).copy()
    T, V = out.shape
    ctx, tok = i32(ctx), i32(tok)
    bt = i32([b[0] for b in bias])
    bv = f32([b[1] for b in bias])
    lib().fnx_o_logit_adjust(_p(out), T, V, _p(ctx), ctx.size, _p(tok), int(last_n), C.c_float(repeat), C.c_float(freq), C.c_float(present),
                             _p(bt), _p(bv), len(bias))
    return out


def lookup(ctx, lk, d1):
    ctx = i32(ctx)
    out = np.empty(max(lk, 1), np.int32)
    match = C.c_int(-1)
    n = lib().fnx_o_lookup(_p(ctx), ctx.size, lk, d1, _p(out), C.byref(match))
    return out[:n].copy(), match.value


def uniform(seed, seq, step, slot):
    return lib().fnx_o_uniform(seed, seq, step, slot)


def philox(ctr, key):
    c = np.asarray(ctr, np.uint32)
    k = np.asarray(key, np.uint32)
    o = np.empty(4, np.uint32)
    lib().fnx_o_philox4x32(_p(c), _p(k), _p(o))
    return o


def make_dist(cand_v, cand_i, s: Sampling):
    cand_v, cand_i = f32(cand_v), i32(cand_i)
    n = cand_v.size
    ids = np.empty(n, np.int32)
    p = np.empty(n, np.float64)
    m = lib().fnx_o_make_dist(_p(cand_v), _p(cand_i), n, C.byref(s), _p(ids), _p(p))
    return ids[:m].copy(), p[:m].copy()


def draw(ids, p, u):
    ids, p = i32(ids), np.ascontiguousarray(p, np.float64)
    return lib().fnx_o_draw(_p(ids), _p(p), ids.size, C.c_double(u))


def accept_greedy(tok, parent, best):
    tok, best = i32(tok), i32(best)
    T = tok.size
    par = None if parent is None else i32(parent)
    path = np.empty(T, np.int32)
    em = np.empty(T, np.int32)
    n = lib().fnx_o_accept_greedy(_p(tok), _p(par), _p(best), T, _p(path), _p(em))
    return n, path[:n].copy(), em[:n].copy()


def accept_sample(cand_v, cand_i, tok, s: Sampling, seed, seq, step, q_ids=None, q_p=None, q_n=None):
    cand_v, cand_i, tok = f32(cand_v), i32(cand_i), i32(tok)
    T = tok.size
    em = np.empty(T, np.int32)
    qi = None if q_ids is None else i32(q_ids)
    qp = None if q_p is None else np.ascontiguousarray(q_p, np.float64)
    qn = None if q_n is None else i32(q_n)
    n = lib().fnx_o_accept_sample(_p(cand_v), _p(cand_i), _p(tok), T, C.byref(s), _p(qi), _p(qp), _p(qn),
                                  C.c_uint64(seed), C.c_uint32(seq), C.c_uint32(step), _p(em))
    return n, em[:n].copy()
