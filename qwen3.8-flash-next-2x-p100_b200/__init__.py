"""Host-side mirror of the reference engine's operator API over the fnx_b200 C ABI.

The product is ``libfnx_b200.so`` (hand-written sm_100a CUDA behind ``include/fnx_b200.h``); this module only
binds it with ctypes so that tests and the benchmark can call the same entry points a C++ host would.  PyTorch is
used for device memory and streams, nothing else.  There is no CPU fallback: if the library has not been built,
``lib()`` raises.

Names follow the reference's ``engine/src/kernels.hpp`` (router_route, moe_gate_up, moe_down, moe_combine,
attn_prep_append, attn, gdn_core, argmax, top_tokens) and ``engine/src/engine.hpp`` (verify, commit, draft).
"""
from __future__ import annotations

import ctypes as C
import pathlib

_HERE = pathlib.Path(__file__).resolve().parent
LIB_PATH = _HERE / "libfnx_b200.so"
HEADER = _HERE.parent / "include" / "fnx_b200.h"
_LIB = None

TOPK_N = 64
MAX_ROWS = 32
JOB_TOK = 4
DENSE_ROWS = 12     # rows of one fnx_dense call (FNX_DENSE_ROWS)
IQ3S_BLOCK = 110


class Job(C.Structure):
    _fields_ = [("w", C.c_int), ("n", C.c_int), ("y", C.c_int * JOB_TOK), ("out", C.c_int * JOB_TOK)]


class Sampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("min_p", C.c_float), ("top_k", C.c_int)]


class ModelConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "n_layer", "hidden", "n_expert", "top_k", "ffn", "n_q_head", "n_kv_head", "head_dim", "n_rot", "gdn_k_head",
        "gdn_v_head", "gdn_head_dim", "vocab", "max_ctx", "max_rows", "attn_every", "ep_rank", "ep_size", "n_seq")] + [
        ("eps", C.c_float), ("rope_base", C.c_float), ("draft_vocab", C.c_int)]


def flash_next_config(**over) -> ModelConfig:
    """The synthetic Qwen3-Next-style model of the benchmark (48 layers, hidden 2048, 512 experts top-10, ffn 512)."""
    d = dict(n_layer=48, hidden=2048, n_expert=512, top_k=10, ffn=512, n_q_head=16, n_kv_head=2, head_dim=256, n_rot=64,
             gdn_k_head=16, gdn_v_head=32, gdn_head_dim=128, vocab=151936, max_ctx=8192, max_rows=8, attn_every=4,
             ep_rank=0, ep_size=1, n_seq=1, eps=1e-6, rope_base=1e7, draft_vocab=0)
    d.update(over)
    return ModelConfig(**d)


_P, _I, _F, _Z, _U64, _U32 = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_uint64, C.c_uint32

_PROTOS = {
    "fnx_last_error": (C.c_char_p, []),
    "fnx_version": (_I, []),
    "fnx_iq3s_bytes": (_Z, [_Z, _Z]),
    "fnx_iq3s_retile": (_I, [_P, _P, _Z, _Z, _P]),
    "fnx_iq3s_untile": (_I, [_P, _P, _Z, _Z, _P]),
    "fnx_iq3s_dequant_tiles": (_I, [_P, _P, _Z, _Z, _P]),
    "fnx_iq3s_quantize": (_I, [_P, _P, _Z, _P]),
    "fnx_fill_normal": (_I, [_P, _Z, _F, _U64, _U32, _P]),
    "fnx_debug_profile_buffer": (_I, [_P]),
    "fnx_dense_rows": (_I, [_I]),
    "fnx_dense": (_I, [_P, _I, _I, _P, _I, _I, _P, _F, _P, _I, _I, _P, _P]),
    "fnx_router_route": (_I, [_P, _P, _P, _F, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P]),
    "fnx_router_rows": (_I, [_P, _P, _P, _F, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P]),
    "fnx_router_rows_scratch_bytes": (_Z, [_I, _I, _I]),
    "fnx_moe_gate_up": (_I, [_P, _Z, _I, _P, _I, _P, _P, _I, _P, _P, _F, _I, _I, _P, _P, _P]),
    "fnx_moe_down": (_I, [_P, _Z, _I, _P, _I, _P, _P, _I, _P, _I, _I, _P, _P, _P]),
    "fnx_moe_combine": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _I, _P]),
    "fnx_moe_combine_image": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _P]),
    "fnx_dense_image_bytes": (_Z, [_I]),
    "fnx_dense_image": (_I, [_P, _I, _I, _P, _I, _I, _F, _P, _I, _I, _P, _P]),
    "fnx_moe_prefill_scratch_bytes": (_Z, [_I, _I, _I, _I, _I]),
    "fnx_dense_prompt_scratch_bytes": (_Z, [_I, _I, _I]),
    "fnx_dense_prompt": (_I, [_P, _I, _I, _P, _I, _P, _F, _P, _I, _I, _P, _P, _P]),
    "fnx_moe_prefill": (_I, [_P, _Z, _P, _Z, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _F, _I, _I, _I, _P, _I, _P, _P, _P]),
    "fnx_argmax_mapped": (_I, [_P, _I, _I, _P, _P, _P, _P, _P]),
    "fnx_attn_prep_append": (_I, [_P, _I, _P, _I, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _F, _F, _P]),
    "fnx_attn_scratch_bytes": (_Z, [_I, _I, _I]),
    "fnx_attn": (_I, [_P, _I, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _P]),
    "fnx_attn_prompt_scratch_bytes": (_Z, [_I, _I, _I]),
    "fnx_attn_prompt": (_I, [_P, _I, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _I, _P]),
    "fnx_attn_static_setup": (_I, []),
    "fnx_attn_static": (_I, [_P, _I, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P]),
    "fnx_gdn_prompt_scratch_bytes": (_Z, [_I, _I, _I, _I]),
    "fnx_gdn_prompt": (_I, [_P, _I, _P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _P, _I, _I, _I, _I, _F, _P, _P]),
    "fnx_gdn_core": (_I, [_P, _I, _P, _I, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _F, _P]),
    "fnx_argmax": (_I, [_P, _I, _I, _P, _P, _P, _P]),
    "fnx_top_tokens": (_I, [_P, _I, _I, _P, _P, _P]),
    "fnx_embed_rows": (_I, [_P, _P, _I, _I, _P, _P]),
    "fnx_mtp_input": (_I, [_P, _P, _P, _P, _P, _F, _P, _I, _P, _I, _I, _P, _P, _P, _P]),
    "fnx_rmsnorm": (_I, [_P, _P, _P, _I, _I, _F, _P]),
    "fnx_lookup_draft": (_I, [_P, _P, _I, _P, _P, _P, _P]),
    "fnx_accept_greedy": (_I, [_P, _P, _P, _I, _P, _P]),
    "fnx_accept_sample": (_I, [_P, _P, _P, _I, Sampling, _P, _P, _P, _U64, _U32, _P, _P, _P]),
    "fnx_engine_create": (_I, [C.POINTER(ModelConfig), C.POINTER(_P)]),
    "fnx_engine_destroy": (None, [_P]),
    "fnx_engine_init_synthetic": (_I, [_P, _U64, _F]),
    "fnx_engine_device_bytes": (_Z, [_P]),
    "fnx_engine_tensor": (_P, [_P, C.c_char_p, C.POINTER(_Z)]),
    "fnx_engine_reset": (_I, [_P, _I]),
    "fnx_engine_verify": (_I, [_P, _I, _P, _P, _I, _P]),
    "fnx_engine_prompt": (_I, [_P, _I, _P, _I]),
    "fnx_engine_verify_lanes_rows": (_I, [_P, _I, _P, _P, _P, _P]),
    "fnx_plan_rows": (_I, [_I, _P, _P, _P, _I, C.c_double, _P, _P, _P]),
    "fnx_engine_prompt_timing": (_I, [_P, _I, _P]),
    "fnx_engine_state_bytes": (_Z, [_P, _I, _I]),
    "fnx_engine_save_state": (_I, [_P, _I, _I, _P, _Z]),
    "fnx_engine_load_state": (_I, [_P, _I, _P, _Z]),
    "fnx_engine_commit": (_I, [_P, _I, _P, _I]),
    "fnx_engine_draft": (_I, [_P, _I, _I, _P]),
    "fnx_engine_last_ms": (_F, [_P]),
    "fnx_engine_counters": (_I, [_P, _P]),
    "fnx_engine_error_bits": (_I, [_P, _P]),
    "fnx_commit": (_I, [_P, _P, _I, _I, _P, _I, _P, _P, _I, _P]),
    "fnx_engine_set_wait_limit": (_I, [_P, C.c_uint]),
    "fnx_engine_ep_open_loopback": (_I, [_P]),
    "fnx_engine_verify_lanes": (_I, [_P, _I, _P, _P, _I, _P]),
    "fnx_engine_commit_lanes": (_I, [_P, _I, _P, _P]),
    "fnx_engine_draft_lanes": (_I, [_P, _I, _P, _I, _P]),
    "fnx_engine_set_position": (_I, [_P, _I, _I]),
    "fnx_attn_prep_append_lanes": (_I, [_P, _I, _P, _I, _P, _I, _P, _P, _P, _P, _Z, _I, _I, _I, _I, _I, _I, _P, _P, _P, _F, _F, _P]),
    "fnx_attn_lanes": (_I, [_P, _I, _P, _P, _Z, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P]),
    "fnx_gdn_core_lanes": (_I, [_P, _I, _P, _I, _P, _Z, _P, _P, _P, _P, _P, _Z, _P, _I, _P, _P, _I, _I, _P, _I, _I, _I, _F, _P]),
    "fnx_accept_greedy_lanes": (_I, [_P, _P, _P, _I, _P, _P]),
    "fnx_accept_sample_lanes": (_I, [_P, _P, _P, Sampling, _U64, _P, _P, _I, _I, _P, _P, _P]),
    "fnx_engine_pos": (_I, [_P, _I]),
    "fnx_engine_stream": (_P, [_P]),
    "fnx_comm_unique_id": (_I, [_P]),
    "fnx_engine_comm_init": (_I, [_P, _P, _I, _I]),
    "fnx_allreduce": (_I, [_P, _P, _Z, _P]),
    "fnx_engine_set_sampling": (_I, [_P, _P, _U64]),
    "fnx_engine_lookup": (_I, [_P, _I, _I, _I, _I, _P, _P]),
    "fnx_engine_ep_handles": (_I, [_P, _P]),
    "fnx_engine_ep_open": (_I, [_P, _P, _I, _I]),
    "fnx_engine_config": (_I, [_P, _P]),
    "fnx_logit_adjust": (_I, [_P, _I, _I, _P, _P, _P, _I, _F, _F, _F, _P, _P, _I, _P]),
    "fnx_engine_set_logit_rules": (_I, [_P, _P]),
    "fnx_gguf_open": (_I, [C.c_char_p, _P]),
    "fnx_gguf_close": (None, [_P]),
    "fnx_gguf_count": (_I, [_P]),
    "fnx_gguf_shards": (_I, [_P]),
    "fnx_gguf_tensor_at": (_I, [_P, _I, _P]),
    "fnx_gguf_find": (_I, [_P, C.c_char_p, _P]),
    "fnx_gguf_num": (_I, [_P, C.c_char_p, _P]),
    "fnx_gguf_str": (_I, [_P, C.c_char_p, _P, _Z]),
    "fnx_gguf_int_array": (_I, [_P, C.c_char_p, _P, _Z, _P]),
    "fnx_gguf_rows_f32": (_I, [_P, C.c_int64, C.c_int64, _P]),
    "fnx_gguf_model_config": (_I, [_P, _P]),
    "fnx_engine_load_gguf": (_I, [_P, _P, _P]),
}
EXPORTS = tuple(_PROTOS)


def lib() -> C.CDLL:
    """The C-ABI library.  Raises when it has not been built: there is no other implementation to fall back to."""
    global _LIB
    if _LIB is None:
        if not LIB_PATH.exists():
            raise ImportError(f"{LIB_PATH} is missing: build it with `python {_HERE / 'build.py'}`")
        L = C.CDLL(str(LIB_PATH))
        for name, (res, args) in _PROTOS.items():
            f = getattr(L, name)
            f.restype = res
            f.argtypes = args
        _LIB = L
    return _LIB


class FnxError(RuntimeError):
    pass


def check(rc: int) -> None:
    if rc != 0:
        raise FnxError(f"fnx_b200 error {rc}: {lib().fnx_last_error().decode()}")


def ptr(t):
    """Device (or host) address of a torch tensor / numpy array, or None."""
    if t is None:
        return None
    if hasattr(t, "data_ptr"):
        return C.c_void_p(t.data_ptr())
    return C.c_void_p(t.ctypes.data)


def _stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


# ------------------------------------------------------------------------------------------------ weights
def iq3s_bytes(rows: int, cols: int) -> int:
    return rows * (cols // 256) * IQ3S_BLOCK


def iq3s_retile(ggml, rows: int, cols: int):
    """GGML IQ3_S blocks (uint8 cuda tensor) -> the device tile layout."""
    import torch
    out = torch.empty(iq3s_bytes(rows, cols), dtype=torch.uint8, device=ggml.device)
    check(lib().fnx_iq3s_retile(ptr(ggml), ptr(out), rows, cols, _stream()))
    return out


def iq3s_untile(tiles, rows: int, cols: int):
    import torch
    out = torch.empty(iq3s_bytes(rows, cols), dtype=torch.uint8, device=tiles.device)
    check(lib().fnx_iq3s_untile(ptr(tiles), ptr(out), rows, cols, _stream()))
    return out


def iq3s_dequant_tiles(tiles, rows: int, cols: int):
    import torch
    out = torch.empty((rows, cols), dtype=torch.float32, device=tiles.device)
    check(lib().fnx_iq3s_dequant_tiles(ptr(tiles), ptr(out), rows, cols, _stream()))
    return out


def iq3s_quantize(w):
    """f32 cuda tensor (numel a multiple of 256) -> GGML IQ3_S blocks (fixture quantiser)."""
    import torch
    out = torch.empty(w.numel() // 256 * IQ3S_BLOCK, dtype=torch.uint8, device=w.device)
    check(lib().fnx_iq3s_quantize(ptr(w), ptr(out), w.numel(), _stream()))
    return out


def fill_normal(out, sigma: float, seed: int, stream_id: int):
    check(lib().fnx_fill_normal(ptr(out), out.numel(), sigma, seed, stream_id, _stream()))
    return out


# ------------------------------------------------------------------------------------------------ operators
def new_err(device="cuda"):
    import torch
    return torch.zeros(1, dtype=torch.int32, device=device)


def dense(W, rows: int, cols: int, x, norm_w=None, eps: float = 1e-6, out=None, accumulate: bool = False, err=None):
    """y[t] (+)= W . x[t] (x optionally RMS-normed with norm_w first): q8s_gemv / mmvq of the reference."""
    import torch
    T = x.shape[0]
    if out is None:
        out = torch.zeros((T, rows), dtype=torch.float32, device=x.device)
    err = new_err(x.device) if err is None else err
    per = lib().fnx_dense_rows(cols)
    for t0 in range(0, T, per):
        nt = min(per, T - t0)
        check(lib().fnx_dense(ptr(W), rows, cols, ptr(x[t0:]), x.stride(0), nt, ptr(norm_w), eps, ptr(out[t0:]), out.stride(0),
                              1 if accumulate else 0, ptr(err), _stream()))
    return out, err


def mtp_input(fc_hid, fc_emb, table_f16, hnorm, enorm, h, tok, eps: float = 1e-6, err=None):
    """The draft layer's input rows: fc_hid . rmsnorm(h) * hnorm + fc_emb . rmsnorm(table[tok]) * enorm
    (mtp_enqueue, engine/src/engine.cu:2103-2113).  Returns (R, emb, err)."""
    import torch
    T, H = h.shape
    R = torch.empty((T, H), dtype=torch.float32, device=h.device)
    emb = torch.empty((T, H), dtype=torch.float32, device=h.device)
    err = new_err(h.device) if err is None else err
    check(lib().fnx_mtp_input(ptr(fc_hid), ptr(fc_emb), ptr(table_f16), ptr(hnorm), ptr(enorm), eps, ptr(h), h.stride(0), ptr(tok), T, H, ptr(emb),
                              ptr(R), ptr(err), _stream()))
    return R, emb, err


def router_route(Wr, x, K: int, norm_w=None, eps: float = 1e-6, e_lo: int = 0, e_hi=None, add_shared: bool = True, err=None):
    import torch
    T, H = x.shape
    E = Wr.shape[0] - 1
    e_hi = E if e_hi is None else e_hi
    dev = x.device
    logits = torch.empty((T, E + 1), dtype=torch.float32, device=dev)
    topi = torch.empty((T, K), dtype=torch.int32, device=dev)
    topw = torch.empty((T, K), dtype=torch.float32, device=dev)
    njobs_max = T * K + (T + JOB_TOK - 1) // JOB_TOK
    jobs = torch.zeros(njobs_max * C.sizeof(Job), dtype=torch.uint8, device=dev)
    njobs = torch.zeros(2, dtype=torch.int32, device=dev)
    err = new_err(dev) if err is None else err
    check(lib().fnx_router_route(ptr(Wr), ptr(x), ptr(norm_w), eps, T, E, H, K, e_lo, e_hi, 1 if add_shared else 0, ptr(logits), ptr(topi),
                                 ptr(topw), ptr(jobs), ptr(njobs), None, ptr(err), _stream()))
    return dict(logits=logits, topi=topi, topw=topw, jobs=jobs, njobs=njobs, njobs_max=njobs_max, err=err)


def moe_experts(Wgu, Wdn, Wsh_gu, Wsh_dn, route, x, F: int, K: int, norm_w=None, eps: float = 1e-6, e_base: int = 0, e_lo: int = 0,
                e_hi=None, add_shared: bool = True):
    """gate|up + SwiGLU, down and combine over a routing result: returns (out [T][H], h, part)."""
    import torch
    T, H = x.shape
    E = route["logits"].shape[1] - 1
    e_hi = E if e_hi is None else e_hi
    P = T * K + T
    gu_stride, dn_stride = iq3s_bytes(2 * F, H), iq3s_bytes(H, F)
    h = torch.zeros((P, F), dtype=torch.float32, device=x.device)
    part = torch.zeros((P, H), dtype=torch.float32, device=x.device)
    out = torch.zeros((T, H), dtype=torch.float32, device=x.device)
    L = lib()
    check(L.fnx_moe_gate_up(ptr(Wgu), gu_stride, e_base, ptr(Wsh_gu), E, ptr(route["jobs"]), ptr(route["njobs"]), route["njobs_max"], ptr(x),
                            ptr(norm_w), eps, H, F, ptr(h), ptr(route["err"]), _stream()))
    check(L.fnx_moe_down(ptr(Wdn), dn_stride, e_base, ptr(Wsh_dn), E, ptr(route["jobs"]), ptr(route["njobs"]), route["njobs_max"], ptr(h), H, F,
                         ptr(part), ptr(route["err"]), _stream()))
    check(L.fnx_moe_combine(ptr(part), ptr(route["topi"]), ptr(route["topw"]), ptr(route["logits"]), T, E, H, K, e_lo, e_hi,
                            1 if add_shared else 0, ptr(out), 0, _stream()))
    return out, h, part


def moe_combine_image(part, route, T: int, E: int, H: int, K: int, R, next_norm_w):
    """R += the weighted expert outputs (fnx_moe_combine, accumulating); returns the image of rmsnorm(R) * next_norm_w."""
    import torch
    L = lib()
    img = torch.zeros(((T + DENSE_ROWS - 1) // DENSE_ROWS) * L.fnx_dense_image_bytes(H), dtype=torch.uint8, device=R.device)
    check(L.fnx_moe_combine_image(ptr(part), ptr(route["topi"]), ptr(route["topw"]), ptr(route["logits"]), T, E, H, K, ptr(R), ptr(img),
                                  ptr(next_norm_w), _stream()))
    return img


def dense_prompt(W, rows: int, cols: int, x, norm_w=None, eps: float = 1e-6, out=None, accumulate: bool = False, err=None):
    """fnx_dense for any number of rows, on the tensor cores: y [T][rows] (+)= W . x[t]."""
    import torch
    T = x.shape[0]
    if out is None:
        out = torch.zeros((T, rows), dtype=torch.float32, device=x.device)
    err = new_err(x.device) if err is None else err
    L = lib()
    scratch = torch.empty(L.fnx_dense_prompt_scratch_bytes(T, rows, cols), dtype=torch.uint8, device=x.device)
    check(L.fnx_dense_prompt(ptr(W), rows, cols, ptr(x), T, ptr(norm_w), eps, ptr(out), out.stride(0), 1 if accumulate else 0, ptr(scratch), ptr(err),
                             _stream()))
    return out, err


def dense_image(W, rows: int, cols: int, img, T: int, normed: bool = True, eps: float = 1e-6, err=None):
    """fnx_dense over rows given as the image a producer left (T rows, in calls of DENSE_ROWS): y [T][rows]."""
    import torch
    y = torch.empty((T, rows), dtype=torch.float32, device=img.device)
    err = new_err(img.device) if err is None else err
    L = lib()
    stride = L.fnx_dense_image_bytes(cols)
    for t0 in range(0, T, DENSE_ROWS):
        nt = min(DENSE_ROWS, T - t0)
        check(L.fnx_dense_image(ptr(W), rows, cols, img.data_ptr() + (t0 // DENSE_ROWS) * stride, nt, 1 if normed else 0, eps, y.data_ptr() + t0 * rows * 4,
                                rows, 0, ptr(err), _stream()))
    return y


def router_rows(Wr, x, K: int, norm_w=None, eps: float = 1e-6, tensor_cores: bool = True):
    """The prompt pass's router over any number of rows in one call: (topi, topw, logits).  tensor_cores: give the call its
    scratch, so that 1,024 rows or more go through the split-f16 product."""
    import torch
    T, H = x.shape
    E = Wr.shape[0] - 1
    logits = torch.empty((T, E + 1), dtype=torch.float32, device=x.device)
    topi = torch.empty((T, K), dtype=torch.int32, device=x.device)
    topw = torch.empty((T, K), dtype=torch.float32, device=x.device)
    err = new_err(x.device)
    scratch = torch.empty(lib().fnx_router_rows_scratch_bytes(T, E, H), dtype=torch.uint8, device=x.device) if tensor_cores else None
    check(lib().fnx_router_rows(ptr(Wr), ptr(x), ptr(norm_w), eps, T, E, H, K, ptr(logits), ptr(topi), ptr(topw), ptr(scratch), ptr(err), _stream()))
    if int(err.item()):
        raise FnxError(f"fnx_router_rows: device error bits {int(err.item()):#x}")
    return topi, topw, logits


class RowCost(C.Structure):
    _fields_ = [("row_lo", C.c_double), ("row_hi", C.c_double), ("chain_ms", C.c_double), ("knee", C.c_int)]


LANE_ROWS = 5


def plan_rows(avail, reach, chain, max_rows: int, base_ms: float, row_lo: float, row_hi: float, chain_ms: float, knee: int):
    """fnx_plan_rows: (drafts per lane, expected tokens per ms).  reach[i] lists lane i's reach probabilities."""
    n = len(avail)
    flat = []
    for r in reach:
        r = list(r)[:LANE_ROWS - 1]
        flat += r + [0.0] * (LANE_ROWS - 1 - len(r))
    out = (C.c_int * n)()
    rate = C.c_double(0.0)
    cost = RowCost(row_lo, row_hi, chain_ms, knee)
    check(lib().fnx_plan_rows(n, (C.c_int * n)(*avail), (C.c_double * len(flat))(*flat), (C.c_int * n)(*[1 if c else 0 for c in chain]), max_rows, base_ms,
                              C.byref(cost), out, C.byref(rate)))
    return list(out), float(rate.value)


def route_rows(Wr, x, K: int, norm_w=None, eps: float = 1e-6):
    """Routing of any number of rows (windows of MAX_ROWS through fnx_router_route): (topi, topw, logits)."""
    import torch
    T = x.shape[0]
    parts = [router_route(Wr, x[t0:t0 + MAX_ROWS].contiguous(), K, norm_w=norm_w, eps=eps) for t0 in range(0, T, MAX_ROWS)]
    return (torch.cat([p["topi"] for p in parts]).contiguous(), torch.cat([p["topw"] for p in parts]).contiguous(),
            torch.cat([p["logits"] for p in parts]).contiguous())


def moe_prefill(Wgu, Wdn, Wsh_gu, Wsh_dn, topi, topw, logits, x, F: int, norm_w=None, eps: float = 1e-6, e_base: int = 0, e_lo: int = 0,
                e_hi=None, add_shared: bool = True, out=None, accumulate: bool = False, scratch=None, err=None):
    """fnx_moe_prefill: the MoE block of T rows with token groups per expert on the tensor cores; returns out [T][H]."""
    import torch
    T, H = x.shape
    K = topi.shape[1]
    E = logits.shape[1] - 1
    e_hi = E if e_hi is None else e_hi
    if out is None:
        out = torch.zeros((T, H), dtype=torch.float32, device=x.device)
    if scratch is None:
        scratch = torch.empty(lib().fnx_moe_prefill_scratch_bytes(T, K, E, H, F), dtype=torch.uint8, device=x.device)
    err = new_err(x.device) if err is None else err
    check(lib().fnx_moe_prefill(ptr(Wgu), iq3s_bytes(2 * F, H), ptr(Wdn), iq3s_bytes(H, F), ptr(Wsh_gu), ptr(Wsh_dn), e_base, E, K, e_lo, e_hi,
                                1 if add_shared else 0, ptr(topi), ptr(topw), ptr(logits), ptr(x), ptr(norm_w), eps, T, H, F, ptr(out),
                                1 if accumulate else 0, ptr(scratch), ptr(err), _stream()))
    return out, err


def attn_prep_append(qg, k, v, q_norm, k_norm, kc, vc, pos0, depth=None, nrot: int = 64, eps: float = 1e-6, rope_base: float = 1e7):
    """In place on qg [T][nq][2 hd] and k [T][nkv][hd]; appends f16 rows to kc / vc [rows][nkv][hd]."""
    T, nq, hd2 = qg.shape
    nkv, hd = k.shape[1], k.shape[2]
    check(lib().fnx_attn_prep_append(ptr(qg), nq * hd2, ptr(k), nkv * hd, ptr(v), nkv * hd, ptr(q_norm), ptr(k_norm), ptr(kc), ptr(vc), T, nq,
                                     nkv, hd, nrot, ptr(pos0), ptr(depth), eps, rope_base, _stream()))


def attn(qg, kc, vc, pos0, parent=None, scratch=None):
    import torch
    T, nq, hd2 = qg.shape
    nkv, hd = kc.shape[1], kc.shape[2]
    out = torch.empty((T, nq, hd), dtype=torch.float32, device=qg.device)
    if scratch is None:
        scratch = torch.empty(lib().fnx_attn_scratch_bytes(T, nq, hd), dtype=torch.uint8, device=qg.device)
    check(lib().fnx_attn(ptr(qg), nq * hd2, ptr(kc), ptr(vc), ptr(out), T, nq, nkv, hd, ptr(pos0), ptr(parent), ptr(scratch), _stream()))
    return out


def attn_prompt(qg, kc, vc, pos0, mma_sync: bool = False, err=None):
    """Attention of a prompt's rows (a chain of any length) over the cache: fnx_attn_prompt (mma_sync: the twelve-row form)."""
    import torch
    T, nq, hd2 = qg.shape
    nkv, hd = kc.shape[1], kc.shape[2]
    out = torch.empty((T, nq, hd), dtype=torch.float32, device=qg.device)
    L = lib()
    scratch = torch.empty(L.fnx_attn_prompt_scratch_bytes(T, nq, hd), dtype=torch.uint8, device=qg.device)
    err = new_err(qg.device) if err is None else err
    check(L.fnx_attn_prompt(ptr(qg), nq * hd2, ptr(kc), ptr(vc), ptr(out), T, nq, nkv, hd, ptr(pos0), ptr(scratch), ptr(err), int(mma_sync), _stream()))
    if int(err.item()):
        raise FnxError(f"fnx_attn_prompt: device error bits {int(err.item()):#x}")
    return out


def attn_static(qg, kc, vc, pos0, parent=None):
    """fnx_attn_static: attention whose split partials live in the library's built-in device array (nothing is allocated
    by the library; `out` is the caller's)."""
    import torch
    T, nq, hd2 = qg.shape
    nkv, hd = kc.shape[1], kc.shape[2]
    out = torch.empty((T, nq, hd), dtype=torch.float32, device=qg.device)
    check(lib().fnx_attn_static(ptr(qg), nq * hd2, ptr(kc), ptr(vc), ptr(out), T, nq, nkv, hd, ptr(pos0), ptr(parent), _stream()))
    return out


def gdn_core(qkvz, ab, hist_pool, convw, dt, a, nw, S_pool, cur, parent, nk: int, nv: int, hs: int = 128, eps: float = 1e-6):
    import torch
    T = qkvz.shape[0]
    y = torch.empty((T, nv * hs), dtype=torch.float32, device=qkvz.device)
    check(lib().fnx_gdn_core(ptr(qkvz), qkvz.stride(0), ptr(ab), ab.stride(0), ptr(hist_pool), ptr(convw), ptr(dt), ptr(a), ptr(nw), ptr(S_pool),
                             ptr(cur), S_pool.shape[0], ptr(parent), ptr(y), nk, nv, hs, T, eps, _stream()))
    return y


def gdn_prompt(qkvz, ab, hist_pool, convw, dt, a, nw, S_pool, cur: int, nk: int, nv: int, hs: int = 128, eps: float = 1e-6):
    """The DeltaNet core over a prompt's rows (any number, a chain, every row kept) from state slot `cur`; the last row's
    state and history land in slot (cur + T) % NS."""
    import torch
    T = qkvz.shape[0]
    y = torch.empty((T, nv * hs), dtype=torch.float32, device=qkvz.device)
    L = lib()
    scratch = torch.empty(L.fnx_gdn_prompt_scratch_bytes(T, nk, nv, hs), dtype=torch.uint8, device=qkvz.device)
    check(L.fnx_gdn_prompt(ptr(qkvz), qkvz.stride(0), ptr(ab), ab.stride(0), ptr(hist_pool), ptr(convw), ptr(dt), ptr(a), ptr(nw), ptr(S_pool), cur,
                           S_pool.shape[0], ptr(y), nk, nv, hs, T, eps, ptr(scratch), _stream()))
    return y


def argmax(logits, err=None):
    import torch
    T, V = logits.shape
    bi = torch.empty(T, dtype=torch.int32, device=logits.device)
    bv = torch.empty(T, dtype=torch.float32, device=logits.device)
    err = new_err(logits.device) if err is None else err
    check(lib().fnx_argmax(ptr(logits), T, V, ptr(bi), ptr(bv), ptr(err), _stream()))
    return bi, bv, err


def top_tokens(logits):
    import torch
    T, V = logits.shape
    ov = torch.empty((T, TOPK_N), dtype=torch.float32, device=logits.device)
    oi = torch.empty((T, TOPK_N), dtype=torch.int32, device=logits.device)
    check(lib().fnx_top_tokens(ptr(logits), T, V, ptr(ov), ptr(oi), _stream()))
    return ov, oi


def lookup_draft(ctx, n, lk: int, d1=None):
    """ctx int32 cuda tensor, n int32[1] (tokens in ctx), d1 int32[1] or None -> (drafts list, match)."""
    import torch
    out = torch.zeros(MAX_ROWS, dtype=torch.int32, device=ctx.device)
    out_n = torch.zeros(2, dtype=torch.int32, device=ctx.device)
    check(lib().fnx_lookup_draft(ptr(ctx), ptr(n), lk, ptr(d1), ptr(out), ptr(out_n), _stream()))
    cnt, match = out_n.tolist()
    return out[:cnt].tolist(), match


def _unpack_result(result):
    r = result.tolist()
    n = r[0]
    return n, r[1:1 + n], r[1 + MAX_ROWS:1 + MAX_ROWS + n]


def accept_greedy(tok, parent, best):
    import torch
    result = torch.zeros(1 + 2 * MAX_ROWS, dtype=torch.int32, device=tok.device)
    check(lib().fnx_accept_greedy(ptr(tok), ptr(parent), ptr(best), tok.numel(), ptr(result), _stream()))
    return _unpack_result(result)


def accept_sample(cand_v, cand_i, tok, s: Sampling, seed: int, seq: int, step, q_ids=None, q_p=None, q_n=None):
    import torch
    result = torch.zeros(1 + 2 * MAX_ROWS, dtype=torch.int32, device=tok.device)
    check(lib().fnx_accept_sample(ptr(cand_v), ptr(cand_i), ptr(tok), tok.numel(), s, ptr(q_ids), ptr(q_p), ptr(q_n), seed, seq, ptr(step),
                                  ptr(result), _stream()))
    return _unpack_result(result)


# ------------------------------------------------------------------------------------------------ engine
class LogitRules(C.Structure):
    _fields_ = [("repeat", C.c_float), ("freq", C.c_float), ("present", C.c_float), ("last_n", C.c_int), ("bias_tok", C.c_void_p),
                ("bias_val", C.c_void_p), ("bias_n", C.c_int)]


def logit_adjust(logits, ctx=None, ctx_n=None, tok=None, last_n: int = 0, repeat: float = 1.0, freq: float = 0.0, present: float = 0.0,
                 bias_tok=None, bias_val=None):
    """In place on logits [T][V]: the logit_bias list, then the penalties over each row's window (k_topk_rows' first half)."""
    T, V = logits.shape
    check(lib().fnx_logit_adjust(ptr(logits), T, V, ptr(ctx), ptr(ctx_n), ptr(tok), last_n, repeat, freq, present, ptr(bias_tok), ptr(bias_val),
                                 0 if bias_tok is None else bias_tok.numel(), _stream()))
    return logits


class GgufTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("type", C.c_uint32), ("n_dims", C.c_int), ("ne", C.c_int64 * 4), ("data", C.c_void_p),
                ("bytes", C.c_size_t), ("shard", C.c_int), ("offset", C.c_uint64)]


class Gguf:
    """The GGUF reader of the C ABI (fnx::Gguf, engine/src/gguf.hpp:47-95): host only, the file stays mapped until close()."""

    def __init__(self, path):
        self._h = C.c_void_p()
        check(lib().fnx_gguf_open(str(path).encode(), C.byref(self._h)))

    def close(self):
        if self._h:
            lib().fnx_gguf_close(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __len__(self):
        return lib().fnx_gguf_count(self._h)

    def shards(self) -> int:
        return lib().fnx_gguf_shards(self._h)

    def tensor_at(self, i: int) -> GgufTensor:
        t = GgufTensor()
        check(lib().fnx_gguf_tensor_at(self._h, i, C.byref(t)))
        return t

    def find(self, name: str):
        t = GgufTensor()
        return t if lib().fnx_gguf_find(self._h, name.encode(), C.byref(t)) else None

    def num(self, key: str):
        v = C.c_double()
        return v.value if lib().fnx_gguf_num(self._h, key.encode(), C.byref(v)) else None

    def str(self, key: str):
        buf = C.create_string_buffer(4096)
        return buf.value.decode() if lib().fnx_gguf_str(self._h, key.encode(), buf, 4096) else None

    def int_array(self, key: str):
        n = C.c_size_t()
        if not lib().fnx_gguf_int_array(self._h, key.encode(), None, 0, C.byref(n)):
            return None
        out = (C.c_int64 * max(n.value, 1))()
        lib().fnx_gguf_int_array(self._h, key.encode(), out, n.value, C.byref(n))
        return list(out[:n.value])

    def rows_f32(self, t: GgufTensor, row0: int = 0, n_rows=None):
        import numpy as np
        rows = t.ne[1] * t.ne[2] * t.ne[3]
        n_rows = rows - row0 if n_rows is None else n_rows
        out = np.empty((n_rows, t.ne[0]), dtype=np.float32)
        check(lib().fnx_gguf_rows_f32(C.byref(t), row0, n_rows, out.ctypes.data_as(C.c_void_p)))
        return out

    def raw(self, t: GgufTensor) -> bytes:
        return C.string_at(t.data, t.bytes)

    def model_config(self, **runtime) -> ModelConfig:
        """The file's architecture with the caller's run-time fields (max_ctx, max_rows, n_seq, ep_rank, ep_size)."""
        d = dict(max_ctx=8192, max_rows=8, ep_rank=0, ep_size=1, n_seq=1)
        d.update(runtime)
        cfg = ModelConfig(**d)
        check(lib().fnx_gguf_model_config(self._h, C.byref(cfg)))
        return cfg


class Engine:
    """Engine::verify / commit / draft of the reference (engine/src/engine.hpp:50-229) over the C ABI."""

    def __init__(self, cfg: ModelConfig):
        self.cfg = cfg
        self._h = C.c_void_p()
        check(lib().fnx_engine_create(C.byref(cfg), C.byref(self._h)))

    def close(self):
        if self._h:
            lib().fnx_engine_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def init_synthetic(self, seed: int = 0, sigma: float = 0.02):
        check(lib().fnx_engine_init_synthetic(self._h, seed, sigma))

    def load_gguf(self, g: Gguf) -> int:
        """Fills the weights from a GGUF file; returns how many tensors had to be quantised to IQ3_S on the way."""
        n = C.c_int(0)
        check(lib().fnx_engine_load_gguf(self._h, g._h, C.byref(n)))
        return n.value

    def config(self) -> ModelConfig:
        cfg = ModelConfig()
        check(lib().fnx_engine_config(self._h, C.byref(cfg)))
        return cfg

    def device_bytes(self) -> int:
        return lib().fnx_engine_device_bytes(self._h)

    def tensor(self, name: str, dtype, shape=None):
        """A torch view of one of the engine's device tensors (no copy)."""
        import torch
        nbytes = C.c_size_t(0)
        p = lib().fnx_engine_tensor(self._h, name.encode(), C.byref(nbytes))
        if not p:
            raise KeyError(name)
        n = nbytes.value // torch.empty(0, dtype=dtype).element_size()

        class _Holder:
            pass
        h = _Holder()
        h.__cuda_array_interface__ = {"shape": (n,), "typestr": {torch.float32: "<f4", torch.int32: "<i4", torch.uint8: "|u1", torch.int64: "<i8",
                                                                 torch.float16: "<f2"}[dtype], "data": (p, False), "version": 2}
        t = torch.as_tensor(h, device="cuda")
        return t if shape is None else t.view(shape)

    def reset(self, seq: int = 0):
        check(lib().fnx_engine_reset(self._h, seq))

    def verify(self, tokens, parents=None, seq: int = 0, want_result: bool = True):
        T = len(tokens)
        tok = (C.c_int * T)(*tokens)
        par = (C.c_int * T)(*parents) if parents is not None else None
        res = (C.c_int * (1 + 2 * MAX_ROWS))() if want_result else None
        check(lib().fnx_engine_verify(self._h, seq, tok, par, T, res))
        if not want_result:
            return None
        n = res[0]
        return n, list(res[1:1 + n]), list(res[1 + MAX_ROWS:1 + MAX_ROWS + n])

    def commit(self, path, seq: int = 0):
        n = len(path)
        check(lib().fnx_engine_commit(self._h, seq, (C.c_int * n)(*path), n))

    def draft(self, k: int, seq: int = 0):
        out = (C.c_int * k)()
        check(lib().fnx_engine_draft(self._h, seq, k, out))
        return list(out)

    def set_sampling(self, sampling=None, seed: int = 0):
        """Sampling (an fnx Sampling struct) or None for greedy windows."""
        check(lib().fnx_engine_set_sampling(self._h, C.byref(sampling) if sampling is not None else None, seed))

    def set_logit_rules(self, last_n: int = 0, repeat: float = 1.0, freq: float = 0.0, present: float = 0.0, bias=()):
        """The request's penalties and logit_bias ((token, bias) pairs) for the following windows; no arguments: none."""
        if last_n <= 0 and not bias:
            check(lib().fnx_engine_set_logit_rules(self._h, None))
            return
        bt = (C.c_int * max(len(bias), 1))(*[int(b[0]) for b in bias])
        bv = (C.c_float * max(len(bias), 1))(*[float(b[1]) for b in bias])
        r = LogitRules(repeat, freq, present, last_n, C.cast(bt, C.c_void_p), C.cast(bv, C.c_void_p), len(bias))
        check(lib().fnx_engine_set_logit_rules(self._h, C.byref(r)))

    def lookup(self, lk: int, d1: int = -1, root: int = -1, seq: int = 0):
        out, n = (C.c_int * MAX_ROWS)(), C.c_int()
        check(lib().fnx_engine_lookup(self._h, seq, lk, d1, root, out, C.byref(n)))
        return list(out[:n.value])

    def verify_lanes(self, seqs, rows_of_tokens, want_result: bool = True):
        """One window of several sequences' rows (a chain of equal length per sequence): per lane (n, path, emitted)."""
        import ctypes as C
        L, T = len(seqs), len(rows_of_tokens[0])
        assert all(len(r) == T for r in rows_of_tokens) and len(rows_of_tokens) == L
        sq = (C.c_int * L)(*seqs)
        tok = (C.c_int * (L * T))(*[t for r in rows_of_tokens for t in r])
        W = 1 + 2 * MAX_ROWS
        res = (C.c_int * (L * W))() if want_result else None
        check(lib().fnx_engine_verify_lanes(self._h, L, sq, tok, T, res))
        if not want_result:
            return None
        out = []
        for j in range(L):
            r = res[j * W:(j + 1) * W]
            out.append((r[0], list(r[1:1 + r[0]]), list(r[1 + MAX_ROWS:1 + MAX_ROWS + r[0]])))
        return out

    def verify_lanes_rows(self, seqs, rows_of_tokens):
        """One window of several sequences' chains of their own lengths: per lane (n, path, emitted)."""
        import ctypes as C
        L = len(seqs)
        rows = [len(r) for r in rows_of_tokens]
        T = sum(rows)
        W = 1 + 2 * MAX_ROWS
        res = (C.c_int * (L * W))()
        check(lib().fnx_engine_verify_lanes_rows(self._h, L, (C.c_int * L)(*seqs), (C.c_int * L)(*rows), (C.c_int * T)(*[t for r in rows_of_tokens for t in r]), res))
        out = []
        for j in range(L):
            r = res[j * W:(j + 1) * W]
            out.append((r[0], list(r[1:1 + r[0]]), list(r[1 + MAX_ROWS:1 + MAX_ROWS + r[0]])))
        return out

    def commit_lanes(self, seqs, keep):
        import ctypes as C
        L = len(seqs)
        check(lib().fnx_engine_commit_lanes(self._h, L, (C.c_int * L)(*seqs), (C.c_int * L)(*keep)))

    def draft_lanes(self, seqs, k: int):
        import ctypes as C
        L = len(seqs)
        out = (C.c_int * (L * k))()
        check(lib().fnx_engine_draft_lanes(self._h, L, (C.c_int * L)(*seqs), k, out))
        return [list(out[j * k:(j + 1) * k]) for j in range(L)]

    def set_position(self, seq: int, pos: int):
        check(lib().fnx_engine_set_position(self._h, seq, pos))

    def error_bits(self) -> int:
        import ctypes as C
        v = C.c_uint(0)
        check(lib().fnx_engine_error_bits(self._h, C.byref(v)))
        return int(v.value)

    def counters(self):
        """(kernels launched through graphs, routed expert jobs, router calls) since creation."""
        out = (C.c_ulonglong * 3)()
        check(lib().fnx_engine_counters(self._h, out))
        return tuple(out)

    def last_ms(self) -> float:
        return lib().fnx_engine_last_ms(self._h)

    def pos(self, seq: int = 0) -> int:
        return lib().fnx_engine_pos(self._h, seq)

    def save_state(self, seq: int = 0, kv: bool = True):
        """The sequence's state as a host buffer (a ctypes array) for load_state."""
        import ctypes as C
        n = lib().fnx_engine_state_bytes(self._h, seq, 1 if kv else 0)
        buf = (C.c_uint8 * n)()
        check(lib().fnx_engine_save_state(self._h, seq, 1 if kv else 0, buf, n))
        return buf

    def load_state(self, buf, seq: int = 0):
        check(lib().fnx_engine_load_state(self._h, seq, buf, len(buf)))

    def prompt(self, tokens, seq: int = 0):
        """Reads a prompt on the prompt-sized kernels (fnx_engine_prompt); leaves the engine as after verify + commit."""
        import ctypes as C
        n = len(tokens)
        check(lib().fnx_engine_prompt(self._h, seq, (C.c_int * n)(*tokens), n))

    def prompt_timing(self, on: bool = True):
        """Switches the prompt pass's phase timing; returns the last timed prompt's ms per phase (a dict)."""
        import ctypes as C
        ms = (C.c_float * 6)()
        check(lib().fnx_engine_prompt_timing(self._h, 1 if on else 0, ms))
        return dict(zip(("in_proj", "attention", "deltanet", "out_proj", "router", "experts"), [float(v) for v in ms]))

    def prefill(self, tokens, seq: int = 0):
        """Reads a prompt by running it through chained verify windows and keeping every row."""
        R = self.cfg.max_rows
        for i in range(0, len(tokens), R):
            w = list(tokens[i:i + R])
            self.verify(w, None, seq, want_result=False)
            self.commit(list(range(len(w))), seq)
