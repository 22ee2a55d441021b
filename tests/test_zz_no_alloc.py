"""GPU test of fnx_attn_static, the attention entry point whose split partials live in a built-in device array.

Collected last on purpose (the file name sorts after the others): it must pass alone and after every other test has
used the device.  It compares two calls in a row with fnx_attn (same kernels, same split order: bit-identical) and
with the CPU oracle, checks that the device's free memory does not move across the calls, and checks the size limit.
"""
import numpy as np
import pytest

from helpers import rel_err

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

NQ, NKV, HD, NROT = 16, 2, 256, 64


def _window(F, O, seed, pos0, T, tree):
    rng = np.random.default_rng(seed)
    rows = pos0 + T + 3
    kc = np.zeros((rows, NKV, HD), np.uint16)
    vc = np.zeros((rows, NKV, HD), np.uint16)
    kc[:pos0] = rng.standard_normal((pos0, NKV, HD)).astype(np.float16).view(np.uint16)
    vc[:pos0] = rng.standard_normal((pos0, NKV, HD)).astype(np.float16).view(np.uint16)
    qg = rng.standard_normal((T, NQ, 2 * HD)).astype(np.float32)
    k = rng.standard_normal((T, NKV, HD)).astype(np.float32)
    v = rng.standard_normal((T, NKV, HD)).astype(np.float32)
    qn = (1 + 0.1 * rng.standard_normal(HD)).astype(np.float32)
    kn = (1 + 0.1 * rng.standard_normal(HD)).astype(np.float32)
    parent = depth = None
    if tree:
        parent = [-1] + [int(rng.integers(0, t)) for t in range(1, T)]
        depth = [0] * T
        for t in range(1, T):
            depth[t] = depth[parent[t]] + 1
    cu = lambda a: torch.as_tensor(np.ascontiguousarray(a)).cuda()
    d = dict(qg=cu(qg), kc=cu(kc.view(np.int16)), vc=cu(vc.view(np.int16)), pos=cu(np.array([pos0], np.int32)),
             par=None if parent is None else cu(np.array(parent, np.int32)))
    d_dep = None if depth is None else cu(np.array(depth, np.int32))
    F.attn_prep_append(d["qg"], cu(k), cu(v), cu(qn), cu(kn), d["kc"], d["vc"], d["pos"], d_dep, NROT)
    O.attn_prep_append(qg, k, v, qn, kn, kc, vc, pos0, depth, NROT)
    d["ref"] = O.attn(qg, kc, vc, pos0, parent)
    return d


def test_static_scratch_attention_equals_caller_scratch_attention_twice_in_a_row(F, O):
    assert F.lib().fnx_attn_static_setup() == 0
    a = _window(F, O, 1, 700, 5, False)
    b = _window(F, O, 2, 300, 8, True)      # another shape: the second call reuses the array with a different layout
    want = [F.attn(w["qg"], w["kc"], w["vc"], w["pos"], w["par"]) for w in (a, b)]
    outs = [torch.empty_like(t) for t in want]
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for w, out in zip((a, b), outs):        # back to back on one stream, no synchronisation in between
        T = w["qg"].shape[0]
        F.check(F.lib().fnx_attn_static(F.ptr(w["qg"]), NQ * 2 * HD, F.ptr(w["kc"]), F.ptr(w["vc"]), F.ptr(out), T, NQ, NKV, HD,
                                        F.ptr(w["pos"]), F.ptr(w["par"]), None))
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0
    for w, out, ref in zip((a, b), outs, want):
        assert torch.equal(out, ref)
        assert rel_err(out.cpu().numpy(), w["ref"]) < 2e-3
    # the same window again after the array held another window's partials
    again = F.attn_static(a["qg"], a["kc"], a["vc"], a["pos"], a["par"])
    assert torch.equal(again, want[0])


def test_static_scratch_attention_rejects_windows_beyond_its_array(F):
    T = 32                                  # 32 rows x 16 heads x 74 splits > 16384 partials
    qg = torch.zeros((T, NQ, 2 * HD), device="cuda")
    kc = torch.zeros((T + 8, NKV, HD), dtype=torch.int16, device="cuda")
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(F.FnxError, match="exceed the built-in scratch"):
        F.attn_static(qg, kc, kc, pos)
    assert F.attn(qg, kc, kc, pos).shape == (T, NQ, HD)   # the caller-scratch entry point takes the same window
