"""GPU parity tests: every operator of the verify path through the C ABI against the CPU oracle.

Bars (from the target): routing indices, accepted counts, greedy tokens and every integer/byte result bit-exact;
hidden states and logits within 1e-2 relative (the kernels are far inside that: the tolerances below are the
tighter figures the two-level int8 activations are expected to hold).
"""
import ctypes as C

import numpy as np
import pytest

from helpers import gpu_iq3s_matrix, rel_err

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

TOL_GEMV = 2e-3   # relative to the largest reference magnitude


def dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


# ------------------------------------------------------------------------------------------------ IQ3_S
def test_retile_is_a_permutation_and_decodes_like_the_oracle(F, O):
    rng = np.random.default_rng(10)
    rows, cols = 64, 1024
    blk = rng.integers(0, 256, size=(rows * cols // 256, 110), dtype=np.uint8)
    d = blk[:, :2].view(np.uint16)
    d[(d & 0x7C00) == 0x7C00] &= 0x3FFF   # keep d finite
    g = dev(blk.reshape(-1))
    tiles = F.iq3s_retile(g, rows, cols)
    assert torch.equal(F.iq3s_untile(tiles, rows, cols), g)
    got = F.iq3s_dequant_tiles(tiles, rows, cols).cpu().numpy()
    ref = O.iq3s_dequant(blk).reshape(rows, cols)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    # sorted bytes of a tile equal sorted bytes of its 16 blocks only if nothing was dropped: check sizes too
    assert tiles.numel() == g.numel() == F.iq3s_bytes(rows, cols)


def test_gpu_quantiser_is_bit_identical_to_the_cpu_twin(F, O):
    rng = np.random.default_rng(11)
    w = (rng.standard_normal((96, 2048)) * 0.02).astype(np.float32)
    w[3, :256] = 0.0          # an all-zero block
    w[5, 256:288] = 0.0       # an all-zero sub-block
    got = F.iq3s_quantize(dev(w)).cpu().numpy()
    ref = O.iq3s_quantize(w).reshape(-1)
    assert np.array_equal(got, ref)
    dq = O.iq3s_dequant(got).reshape(w.shape)
    assert np.sqrt(((dq - w) ** 2).mean()) / w.std() < 0.2


# ------------------------------------------------------------------------------------------------ dense GEMV
@pytest.mark.parametrize("rows,cols,T", [(64, 2048, 1), (64, 2048, 5), (128, 512, 4), (256, 512, 8), (32, 4096, 5), (256, 256, 3),
                                         (64, 1024, 7), (9216, 2048, 5), (2048, 4096, 5), (128, 2048, 20), (256, 2048, 12), (2048, 4096, 11),
                                         (64, 1024, 9)])
def test_dense_matches_oracle(F, O, rows, cols, T):
    tiles, ggml = gpu_iq3s_matrix(F, rows, cols, seed=3, stream_id=rows + cols)
    rng = np.random.default_rng(rows + T)
    x = rng.standard_normal((T, cols)).astype(np.float32)
    y, err = F.dense(tiles, rows, cols, dev(x))
    ref = O.iq3s_gemv(ggml, rows, cols, x)
    assert int(err.item()) == 0
    assert rel_err(y.cpu().numpy(), ref) < TOL_GEMV


def test_dense_with_norm_accumulate_and_strides(F, O):
    rows, cols, T = 2048, 2048, 5
    tiles, ggml = gpu_iq3s_matrix(F, rows, cols, seed=4, stream_id=77)
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((T, cols)) * 3.0).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    base = rng.standard_normal((T, rows + 64)).astype(np.float32)
    out = dev(base)
    y, err = F.dense(tiles, rows, cols, dev(x), norm_w=dev(w), eps=1e-6, out=out[:, :rows], accumulate=True)
    ref = base[:, :rows] + O.iq3s_gemv(ggml, rows, cols, O.rmsnorm(x, w, 1e-6))
    assert int(err.item()) == 0
    assert rel_err(out[:, :rows].cpu().numpy(), ref) < TOL_GEMV
    assert np.array_equal(out[:, rows:].cpu().numpy(), base[:, rows:])   # nothing written past the rows


@pytest.mark.parametrize("T", [1, 5, 20])
def test_mtp_input_matches_oracle(F, O, T):
    """The draft layer's input rows against the oracle's composition, and bit-equal to the two dense calls they stand for
    (20 rows: more than one call of the dense form)."""
    import torch
    H, V = 2048, 300
    hid_t, hid_g = gpu_iq3s_matrix(F, H, H, seed=8, stream_id=1)
    emb_t, emb_g = gpu_iq3s_matrix(F, H, H, seed=8, stream_id=2)
    rng = np.random.default_rng(40 + T)
    table = (rng.standard_normal((V, H)) * 0.5).astype(np.float16)
    hn = (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    en = (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    h = (rng.standard_normal((T, H + 32)) * 2.0).astype(np.float32)   # rows with a stride
    tok = rng.integers(0, V, T).astype(np.int32)
    hd = dev(h)[:, :H]
    R, emb, err = F.mtp_input(hid_t, emb_t, dev(table), dev(hn), dev(en), hd, dev(tok))
    assert int(err.item()) == 0
    e32 = table[tok].astype(np.float32)
    assert np.array_equal(emb.cpu().numpy(), e32)
    ref = O.iq3s_gemv(hid_g, H, H, O.rmsnorm(h[:, :H], hn, 1e-6)) + O.iq3s_gemv(emb_g, H, H, O.rmsnorm(e32, en, 1e-6))
    assert rel_err(R.cpu().numpy(), ref) < TOL_GEMV
    two, _ = F.dense(hid_t, H, H, hd, norm_w=dev(hn))
    F.dense(emb_t, H, H, dev(e32), norm_w=dev(en), out=two, accumulate=True)
    assert torch.equal(R, two)


def test_dense_zero_and_huge_inputs(F, O):
    rows, cols = 64, 2048
    tiles, ggml = gpu_iq3s_matrix(F, rows, cols, seed=6, stream_id=5)
    x = np.zeros((2, cols), np.float32)
    x[1, ::7] = 1e4
    y, err = F.dense(tiles, rows, cols, dev(x))
    ref = O.iq3s_gemv(ggml, rows, cols, x)
    assert np.all(y[0].cpu().numpy() == 0.0)
    assert rel_err(y.cpu().numpy(), ref) < TOL_GEMV


@pytest.mark.parametrize("rows,cols,T", [(256, 2048, 300), (208, 1024, 70), (2048, 4096, 513), (208, 1024, 1100), (1616, 2048, 1300)])
def test_dense_prompt_matches_the_decode_product(F, rows, cols, T):
    """The prompt-sized projection (tensor cores, f16 activations) against the decode kernel's product of the same rows: same
    weights, activations rounded to f16 instead of two int8 levels; with the norm, into a strided output, accumulating; a
    feature count that is not a multiple of the 128-feature slab (208).  From 1,024 rows on the product takes the matrix decoded
    to f16 once and both operands by tensor copies: row and feature counts that end inside a tile (1,100 and 1,300; 208 and 1,616)."""
    import torch
    Wt, _ = gpu_iq3s_matrix(F, rows, cols, 3, 77)
    rng = np.random.default_rng(T)
    x = dev(rng.standard_normal((T, cols)).astype(np.float32))
    nw = dev((1.0 + 0.05 * rng.standard_normal(cols)).astype(np.float32))
    want, _ = F.dense(Wt, rows, cols, x, norm_w=nw)
    got, err = F.dense_prompt(Wt, rows, cols, x, norm_w=nw)
    assert int(err.item()) == 0
    assert rel_err(got.cpu().numpy(), want.cpu().numpy()) < 2e-3
    base = dev(rng.standard_normal((T, rows + 16)).astype(np.float32))
    acc = base.clone()
    F.dense_prompt(Wt, rows, cols, x, out=acc[:, :rows], accumulate=True)
    plain, _ = F.dense(Wt, rows, cols, x)
    assert rel_err((acc[:, :rows] - base[:, :rows]).cpu().numpy(), plain.cpu().numpy()) < 2e-3
    assert torch.equal(acc[:, rows:], base[:, rows:])


def test_dense_rows_do_not_depend_on_the_call_they_ride_in(F):
    """A row's product is the same bits alone, among 5 rows and among 12 (one, two or three row groups per call)."""
    import torch
    rows, cols = 512, 2048
    Wt, _ = gpu_iq3s_matrix(F, rows, cols, 3, 41)
    rng = np.random.default_rng(12)
    x = dev(rng.standard_normal((12, cols)).astype(np.float32))
    nw = dev((1.0 + 0.05 * rng.standard_normal(cols)).astype(np.float32))
    y12, _ = F.dense(Wt, rows, cols, x, norm_w=nw)
    y5, _ = F.dense(Wt, rows, cols, x[:5].contiguous(), norm_w=nw)
    y1, _ = F.dense(Wt, rows, cols, x[3:4].contiguous(), norm_w=nw)
    assert torch.equal(y12[:5], y5) and torch.equal(y12[3:4], y1)


def test_dense_rejects_bad_shapes(F):
    tiles = torch.zeros(F.iq3s_bytes(64, 2048), dtype=torch.uint8, device="cuda")
    x = torch.zeros((1, 2048), device="cuda")
    with pytest.raises(F.FnxError):
        F.dense(tiles, 40, 2048, x)          # not a whole number of 16-row tiles
    with pytest.raises(F.FnxError):
        F.dense(tiles, 64, 768, x[:, :768])  # unsupported column count


# ------------------------------------------------------------------------------------------------ MoE
def _moe_fixture(F, E, H, Fn, seed):
    gu_t, gu_g, dn_t, dn_g = [], [], [], []
    for e in range(E):
        t, g = gpu_iq3s_matrix(F, 2 * Fn, H, seed, 1000 + e)
        gu_t.append(t); gu_g.append(g)
        t, g = gpu_iq3s_matrix(F, H, Fn, seed, 5000 + e)
        dn_t.append(t); dn_g.append(g)
    sh_gu_t, sh_gu_g = gpu_iq3s_matrix(F, 2 * Fn, H, seed, 9000)
    sh_dn_t, sh_dn_g = gpu_iq3s_matrix(F, H, Fn, seed, 9001)
    wr = torch.empty((E + 1) * H, dtype=torch.float32, device="cuda")
    F.fill_normal(wr, 0.02, seed, 9002)
    return dict(gu_t=torch.cat(gu_t), dn_t=torch.cat(dn_t), gu_g=np.concatenate(gu_g), dn_g=np.concatenate(dn_g), sh_gu_t=sh_gu_t,
                sh_dn_t=sh_dn_t, sh_gu_g=sh_gu_g, sh_dn_g=sh_dn_g, wr=wr.view(E + 1, H))


def _check_jobs(F, route, T, K, E, topi, e_lo, e_hi, add_shared):
    nj = int(route["njobs"][0].item())
    assert int(route["njobs"][1].item()) == 0
    raw = route["jobs"].cpu().numpy().tobytes()
    jobs = (F.Job * route["njobs_max"]).from_buffer_copy(raw)
    seen = set()
    shared_rows = set()
    for j in range(nj):
        jb = jobs[j]
        assert 1 <= jb.n <= F.JOB_TOK
        for i in range(jb.n):
            if jb.w == E:
                assert jb.out[i] == T * K + jb.y[i]
                shared_rows.add(jb.y[i])
            else:
                assert e_lo <= jb.w < e_hi
                t, k = divmod(jb.out[i], K)
                assert t == jb.y[i] and topi[t, k] == jb.w
                seen.add(jb.out[i])
    want = {t * K + k for t in range(T) for k in range(K) if e_lo <= topi[t, k] < e_hi}
    assert seen == want
    assert shared_rows == (set(range(T)) if add_shared else set())


@pytest.mark.parametrize("E,H,K,T", [(32, 1024, 4, 77), (512, 2048, 10, 300), (512, 2048, 10, 1500), (32, 1024, 4, 1100)])
def test_router_rows_equals_the_window_router(F, E, H, K, T):
    """The prompt pass's router over T rows in one call against fnx_router_route over windows of 32 rows: the same picks wherever
    the K-th and (K + 1)-th logits are not a rounding apart, logits and weights to 1e-6.  From 1,024 rows on the logits are the
    tensor-core product of the split operands: against the f32 walk (scratch = null) and a float64 product."""
    import torch
    rng = np.random.default_rng(E + T)
    wr = dev((0.02 * rng.standard_normal((E + 1, H))).astype(np.float32))
    x = dev(rng.standard_normal((T, H)).astype(np.float32))
    nw = dev((1.0 + 0.05 * rng.standard_normal(H)).astype(np.float32))
    ti, tw, lg = F.router_rows(wr, x, K, norm_w=nw)
    ri, rw, rl = F.route_rows(wr, x, K, norm_w=nw)
    big = T >= 1024
    if big:
        _, _, walk = F.router_rows(wr, x, K, norm_w=nw, tensor_cores=False)
        assert np.abs(walk.cpu().numpy() - rl.cpu().numpy()).max() < 1e-6
        x64 = x.cpu().numpy().astype(np.float64)
        xn = x64 / np.sqrt((x64 * x64).mean(axis=1, keepdims=True) + 1e-6) * nw.cpu().numpy().astype(np.float64)
        ref = xn @ wr.cpu().numpy().astype(np.float64).T
        # the tensor core sums its f32 accumulator by truncation: ~2^-24 of the running sum per step, 384 steps
        assert np.abs(walk.cpu().numpy() - ref).max() < 3e-6 and np.abs(lg.cpu().numpy() - ref).max() < 1e-4
        assert np.abs(lg.cpu().numpy() - ref).mean() < 1e-5
    assert np.abs(lg.cpu().numpy() - rl.cpu().numpy()).max() < (1e-4 if big else 1e-6)
    srt = np.sort(rl.cpu().numpy()[:, :E], axis=1)
    # rows whose K + 1 highest logits lie further apart than the two routers' logits differ: there the picks agree in order too
    clear = np.diff(srt[:, -K - 1:], axis=1).min(axis=1) > (3e-4 if big else 1e-5)
    assert clear.sum() > T // 2
    assert np.array_equal(ti.cpu().numpy()[clear], ri.cpu().numpy()[clear])
    assert np.abs(tw.cpu().numpy()[clear] - rw.cpu().numpy()[clear]).max() < (1e-4 if big else 1e-5)


@pytest.mark.parametrize("E,H,Fn,K,T", [(32, 1024, 256, 4, 3), (64, 2048, 512, 10, 5), (64, 2048, 512, 10, 20)])
def test_moe_block_matches_oracle(F, O, E, H, Fn, K, T):
    fx = _moe_fixture(F, E, H, Fn, seed=21)
    rng = np.random.default_rng(E + T)
    x = rng.standard_normal((T, H)).astype(np.float32)
    nw = (1.0 + 0.05 * rng.standard_normal(H)).astype(np.float32)
    xn = O.rmsnorm(x, nw, 1e-6)
    ref_out, ref_logits, ref_topi, ref_topw = O.moe(fx["wr"].cpu().numpy(), fx["gu_g"], fx["dn_g"], fx["sh_gu_g"], fx["sh_dn_g"], xn, Fn, K)
    route = F.router_route(fx["wr"], dev(x), K, norm_w=dev(nw))
    assert np.array_equal(route["topi"].cpu().numpy(), ref_topi)            # routing indices: bit-exact
    assert rel_err(route["logits"].cpu().numpy(), ref_logits) < 1e-5
    assert np.abs(route["topw"].cpu().numpy() - ref_topw).max() < 1e-5
    _check_jobs(F, route, T, K, E, ref_topi, 0, E, True)
    out, h, part = F.moe_experts(fx["gu_t"], fx["dn_t"], fx["sh_gu_t"], fx["sh_dn_t"], route, dev(x), Fn, K, norm_w=dev(nw))
    assert int(route["err"].item()) == 0
    assert rel_err(out.cpu().numpy(), ref_out) < TOL_GEMV
    # expert-parallel shards add up to the whole (2 ranks), the shared expert counted once
    acc = np.zeros_like(ref_out)
    for r in range(2):
        lo, hi = r * E // 2, (r + 1) * E // 2
        rt = F.router_route(fx["wr"], dev(x), K, norm_w=dev(nw), e_lo=lo, e_hi=hi, add_shared=(r == 0))
        _check_jobs(F, rt, T, K, E, ref_topi, lo, hi, r == 0)
        gu_b, dn_b = F.iq3s_bytes(2 * Fn, H), F.iq3s_bytes(H, Fn)
        o, _, _ = F.moe_experts(fx["gu_t"][lo * gu_b:hi * gu_b], fx["dn_t"][lo * dn_b:hi * dn_b], fx["sh_gu_t"], fx["sh_dn_t"], rt, dev(x), Fn, K,
                                norm_w=dev(nw), e_base=lo, e_lo=lo, e_hi=hi, add_shared=(r == 0))
        ref_r, _, _, _ = O.moe(fx["wr"].cpu().numpy(), fx["gu_g"], fx["dn_g"], fx["sh_gu_g"], fx["sh_dn_g"], xn, Fn, K, e_lo=lo, e_hi=hi,
                               add_shared=(r == 0))
        assert rel_err(o.cpu().numpy(), ref_r) < TOL_GEMV
        acc += o.cpu().numpy()
    assert rel_err(acc, ref_out) < TOL_GEMV


@pytest.mark.parametrize("T", [1, 5, 8, 20])
def test_combine_that_leaves_the_image_gives_the_same_bits(F, T):
    """fnx_moe_combine_image updates the residual like fnx_moe_combine (accumulating), bit for bit, and the image it leaves
    feeds fnx_dense_image the bits fnx_dense computes from the rows themselves; a smaller window after a larger one leaves no
    stale rows behind."""
    import torch
    E, H, Fn, K = 64, 2048, 512, 10
    fx = _moe_fixture(F, E, H, Fn, seed=21)
    rng = np.random.default_rng(100 + T)
    nw = dev((1.0 + 0.05 * rng.standard_normal(H)).astype(np.float32))
    nw2 = dev((1.0 + 0.05 * rng.standard_normal(H)).astype(np.float32))
    Wd = fx["gu_t"]   # any tile matrix with 2048 columns serves as the next projection: expert 0's gate|up (1024 rows)
    rows = 2 * Fn
    L = F.lib()
    for rep in range(2):
        x = dev(rng.standard_normal((T, H)).astype(np.float32))
        R0 = dev(rng.standard_normal((T, H)).astype(np.float32))
        route = F.router_route(fx["wr"], x, K, norm_w=nw)
        out, h, part = F.moe_experts(fx["gu_t"], fx["dn_t"], fx["sh_gu_t"], fx["sh_dn_t"], route, x, Fn, K, norm_w=nw)
        want = R0.clone()
        F.check(L.fnx_moe_combine(F.ptr(part), F.ptr(route["topi"]), F.ptr(route["topw"]), F.ptr(route["logits"]), T, E, H, K, 0, E, 1, F.ptr(want), 1,
                                  None))
        got = R0.clone()
        img = F.moe_combine_image(part, route, T, E, H, K, got, nw2)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        y_img = F.dense_image(Wd, rows, H, img, T)
        y_ref, _ = F.dense(Wd, rows, H, want, norm_w=nw2)
        assert torch.equal(y_img, y_ref)
    if T == 5:   # the image buffer held 8 rows before: the rows of the group that hold nothing now must read as zero
        img8 = torch.full_like(img, 0x55)
        F.check(L.fnx_moe_combine_image(F.ptr(part), F.ptr(route["topi"]), F.ptr(route["topw"]), F.ptr(route["logits"]), T, E, H, K, F.ptr(R0.clone()),
                                        F.ptr(img8), F.ptr(nw2), None))
        got = R0.clone()
        F.check(L.fnx_moe_combine_image(F.ptr(part), F.ptr(route["topi"]), F.ptr(route["topw"]), F.ptr(route["logits"]), T, E, H, K, F.ptr(got), F.ptr(img8),
                                        F.ptr(nw2), None))
        assert torch.equal(F.dense_image(Wd, rows, H, img8, T), y_ref)


_CONFIG0 = {}


def _config0_fixture(F):
    """The first benchmark configuration's MoE block at its full size: hidden 2048, 512 routed experts of width 512
    (N(0, 0.02) from seed 0, quantised to IQ3_S), top-10 + one shared expert; built once per session (700 MB of blocks)."""
    if not _CONFIG0:
        _CONFIG0.update(_moe_fixture(F, 512, 2048, 512, seed=0))
    return _CONFIG0


@pytest.mark.parametrize("T", [5, 20])
def test_config0_moe_block_at_full_size(F, O, T):
    """512 experts, top-10, 5 verify rows (seed 1) and a 20-row tree window: routing indices bit-exact, hidden states within
    the kernels' 2e-3 (the target asks 1e-2); ~50 (T = 5) or ~170 (T = 20) jobs spread over the 148 blocks in several passes,
    expert strides of 1.35 MB; expert-parallel shards of 2, 4 and 8 ranks add up to the whole."""
    E, H, Fn, K = 512, 2048, 512, 10
    fx = _config0_fixture(F)
    x = np.random.default_rng(1).standard_normal((T, H)).astype(np.float32)
    ref_out, ref_logits, ref_topi, ref_topw = O.moe(fx["wr"].cpu().numpy(), fx["gu_g"], fx["dn_g"], fx["sh_gu_g"], fx["sh_dn_g"], x, Fn, K)
    srt = np.sort(ref_logits[:, :E], axis=1)
    assert (srt[:, -K] - srt[:, -K - 1]).min() > 1e-5, "a near-tie at the top-K boundary: pick another seed"
    route = F.router_route(fx["wr"], dev(x), K)
    assert np.array_equal(route["topi"].cpu().numpy(), ref_topi)
    _check_jobs(F, route, T, K, E, ref_topi, 0, E, True)
    out, h, part = F.moe_experts(fx["gu_t"], fx["dn_t"], fx["sh_gu_t"], fx["sh_dn_t"], route, dev(x), Fn, K)
    assert int(route["err"].item()) == 0
    assert rel_err(out.cpu().numpy(), ref_out) < TOL_GEMV
    gu_b, dn_b = F.iq3s_bytes(2 * Fn, H), F.iq3s_bytes(H, Fn)
    for R in (2, 4, 8):
        acc = np.zeros_like(ref_out)
        for r in range(R):
            lo, hi = r * E // R, (r + 1) * E // R
            rt = F.router_route(fx["wr"], dev(x), K, e_lo=lo, e_hi=hi, add_shared=(r == 0))
            o, _, _ = F.moe_experts(fx["gu_t"][lo * gu_b:hi * gu_b], fx["dn_t"][lo * dn_b:hi * dn_b], fx["sh_gu_t"], fx["sh_dn_t"], rt, dev(x), Fn, K,
                                    e_base=lo, e_lo=lo, e_hi=hi, add_shared=(r == 0))
            acc += o.cpu().numpy()
        assert rel_err(acc, ref_out) < TOL_GEMV


def test_prefill_moe_at_full_size_matches_the_decode_path_and_the_oracle(F, O):
    """The prompt-sized MoE block at the benchmark's own size (512 experts of width 512, hidden 2048, top-10) over 16,384 rows:
    ~320 rows per expert, so most experts run two jobs (256 rows + a ragged tail).  Sampled rows against the decode kernels
    (themselves checked against the oracle at this size) and a few against the oracle directly."""
    import torch
    E, H, Fn, K, T = 512, 2048, 512, 10, 16384
    fx = _config0_fixture(F)
    x = torch.randn((T, H), device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))
    topi, topw, logits = F.router_rows(fx["wr"], x, K)
    cnt = torch.bincount(topi.flatten().long(), minlength=E)
    assert int(cnt.max().item()) > 256 and int((cnt > 256).sum().item()) > E // 2      # most experts need a second job
    out, err = F.moe_prefill(fx["gu_t"], fx["dn_t"], fx["sh_gu_t"], fx["sh_dn_t"], topi, topw, logits, x, Fn)
    assert int(err.item()) == 0
    rows = torch.randperm(T, generator=torch.Generator().manual_seed(6))[:40].sort().values.cuda()
    xs = x[rows].contiguous()
    got = out[rows].cpu().numpy()
    dec = []
    for t0 in range(0, 40, 20):
        route = F.router_route(fx["wr"], xs[t0:t0 + 20].contiguous(), K)
        o, _, _ = F.moe_experts(fx["gu_t"], fx["dn_t"], fx["sh_gu_t"], fx["sh_dn_t"], route, xs[t0:t0 + 20].contiguous(), Fn, K)
        assert int(route["err"].item()) == 0
        dec.append(o)
        # (the two routers agree on these rows, or the comparison below means nothing)
        assert torch.equal(route["topi"].sort(dim=1).values, topi[rows[t0:t0 + 20]].sort(dim=1).values)
    assert rel_err(got, torch.cat(dec).cpu().numpy()) < 3e-3
    ref, _, _, _ = O.moe(fx["wr"].cpu().numpy(), fx["gu_g"], fx["dn_g"], fx["sh_gu_g"], fx["sh_dn_g"], xs[:8].cpu().numpy(), Fn, K)
    assert rel_err(got[:8], ref) < 3e-3


def test_router_many_tokens_pick_one_expert(F, O):
    # every row identical: all rows pick the same experts, so jobs split into groups of 4 rows
    E, H, K, T = 32, 1024, 4, 9
    rng = np.random.default_rng(2)
    wr = (rng.standard_normal((E + 1, H)) * 0.02).astype(np.float32)
    x = np.tile(rng.standard_normal((1, H)).astype(np.float32), (T, 1))
    _, ref_topi, _ = O.router(wr, x, K)
    route = F.router_route(dev(wr), dev(x), K)
    assert np.array_equal(route["topi"].cpu().numpy(), ref_topi)
    _check_jobs(F, route, T, K, E, ref_topi, 0, E, True)
    assert int(route["njobs"][0].item()) == K * 3 + 3


@pytest.mark.parametrize("E,H,Fn,K,T", [(16, 512, 256, 4, 200), (32, 2048, 512, 10, 333), (16, 512, 256, 4, 1300), (32, 2048, 512, 10, 1100)])
def test_prefill_moe_on_tensor_cores_matches_oracle(F, O, E, H, Fn, K, T):
    """Token groups per expert through tcgen05.mma (f16 operands, f32 accumulate): jobs of 128 rows and ragged tails,
    experts nobody picked, the shared expert over all rows.  From 1,024 rows on the experts' matrices are decoded to f16 once and
    the grouped products take both operands by tensor copies (rows copied into job order)."""
    fx = _moe_fixture(F, E, H, Fn, seed=23)
    rng = np.random.default_rng(E + T)
    x = rng.standard_normal((T, H)).astype(np.float32)
    nw = (1.0 + 0.05 * rng.standard_normal(H)).astype(np.float32)
    xn = O.rmsnorm(x, nw, 1e-6)
    ref_out, _, ref_topi, _ = O.moe(fx["wr"].cpu().numpy(), fx["gu_g"], fx["dn_g"], fx["sh_gu_g"], fx["sh_dn_g"], xn, Fn, K)
    topi, topw, logits = F.route_rows(fx["wr"], dev(x), K, norm_w=dev(nw))
    assert np.array_equal(topi.cpu().numpy(), ref_topi)
    out, err = F.moe_prefill(fx["gu_t"], fx["dn_t"], fx["sh_gu_t"], fx["sh_dn_t"], topi, topw, logits, dev(x), Fn, norm_w=dev(nw))
    assert int(err.item()) == 0
    # f16 operands: each product term carries 2^-11 relative rounding twice; the sums stay well inside the 1e-2 bar
    assert rel_err(out.cpu().numpy(), ref_out) < 3e-3
    # the decode-sized path gives the same block (first rows)
    route = F.router_route(fx["wr"], dev(x[:5]), K, norm_w=dev(nw))
    small, _, _ = F.moe_experts(fx["gu_t"], fx["dn_t"], fx["sh_gu_t"], fx["sh_dn_t"], route, dev(x[:5]), Fn, K, norm_w=dev(nw))
    assert rel_err(out[:5].cpu().numpy(), small.cpu().numpy()) < 3e-3


# ------------------------------------------------------------------------------------------------ attention
@pytest.mark.parametrize("pos0,T,tree", [(0, 1, False), (37, 5, False), (300, 5, True), (4096, 5, False), (1000, 20, True)])
def test_attention_matches_oracle(F, O, pos0, T, tree):
    nq, nkv, hd, nrot = 16, 2, 256, 64
    rng = np.random.default_rng(pos0 + T)
    rows = pos0 + T + 3
    kc = np.zeros((rows, nkv, hd), np.uint16)
    vc = np.zeros((rows, nkv, hd), np.uint16)
    kc[:pos0] = (rng.standard_normal((pos0, nkv, hd))).astype(np.float16).view(np.uint16)
    vc[:pos0] = (rng.standard_normal((pos0, nkv, hd))).astype(np.float16).view(np.uint16)
    qg = rng.standard_normal((T, nq, 2 * hd)).astype(np.float32)
    k = rng.standard_normal((T, nkv, hd)).astype(np.float32)
    v = rng.standard_normal((T, nkv, hd)).astype(np.float32)
    qn = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    kn = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    parent = depth = None
    if tree:
        parent = [-1] + [int(rng.integers(0, t)) for t in range(1, T)]
        depth = [0] * T
        for t in range(1, T):
            depth[t] = depth[parent[t]] + 1
    d_qg, d_k, d_kc, d_vc = dev(qg), dev(k), dev(kc.view(np.int16)), dev(vc.view(np.int16))
    d_pos = dev(np.array([pos0], np.int32))
    d_par = None if parent is None else dev(np.array(parent, np.int32))
    d_dep = None if depth is None else dev(np.array(depth, np.int32))
    F.attn_prep_append(d_qg, d_k, dev(v), dev(qn), dev(kn), d_kc, d_vc, d_pos, d_dep, nrot)
    out = F.attn(d_qg, d_kc, d_vc, d_pos, d_par)
    O.attn_prep_append(qg, k, v, qn, kn, kc, vc, pos0, depth, nrot)
    ref = O.attn(qg, kc, vc, pos0, parent)
    # the rotary angle is position x frequency in f32 (as the reference computes it): one ulp of the frequency moves the
    # angle by position x 2^-23, so the bar grows with the position
    assert rel_err(d_qg.cpu().numpy(), qg) < 1e-5 + 2.5e-7 * pos0
    # appended cache rows: f16 of values that agree to ~1e-6, so at most one f16 step apart, and almost all equal
    got_k = d_kc.cpu().numpy().view(np.uint16)[pos0:pos0 + T].astype(np.int32)
    assert np.abs(got_k - kc[pos0:pos0 + T].astype(np.int32)).max() <= 1 + pos0 // 1000
    assert (got_k != kc[pos0:pos0 + T]).mean() < 1e-3 + 1e-5 * pos0
    assert np.array_equal(d_vc.cpu().numpy().view(np.uint16)[pos0:pos0 + T], vc[pos0:pos0 + T])
    assert rel_err(out.cpu().numpy(), ref) < 2e-3


@pytest.mark.parametrize("pos0,T", [(0, 1), (0, 50), (333, 77), (5000, 13)])
def test_prompt_attention_matches_windows(F, O, pos0, T):
    """A prompt's rows in one call (twelve rows per block, f16 queries, no splits) against chained windows of the window form:
    the same cache rows appended, outputs to the f16-query tolerance."""
    nq, nkv, hd, nrot = 16, 2, 256, 64
    rng = np.random.default_rng(pos0 * 7 + T)
    rows = pos0 + T + 3
    kc = np.zeros((rows, nkv, hd), np.uint16)
    vc = np.zeros((rows, nkv, hd), np.uint16)
    kc[:pos0] = (rng.standard_normal((pos0, nkv, hd))).astype(np.float16).view(np.uint16)
    vc[:pos0] = (rng.standard_normal((pos0, nkv, hd))).astype(np.float16).view(np.uint16)
    qg = rng.standard_normal((T, nq, 2 * hd)).astype(np.float32)
    k = rng.standard_normal((T, nkv, hd)).astype(np.float32)
    v = rng.standard_normal((T, nkv, hd)).astype(np.float32)
    qn = dev((1 + 0.1 * rng.standard_normal(hd)).astype(np.float32))
    kn = dev((1 + 0.1 * rng.standard_normal(hd)).astype(np.float32))
    # windows of 32 rows
    w_kc, w_vc = dev(kc.view(np.int16)), dev(vc.view(np.int16))
    outs = []
    for t0 in range(0, T, 32):
        nt = min(32, T - t0)
        q_w, pos = dev(qg[t0:t0 + nt]), dev(np.array([pos0 + t0], np.int32))
        F.attn_prep_append(q_w, dev(k[t0:t0 + nt]), dev(v[t0:t0 + nt]), qn, kn, w_kc, w_vc, pos, None, nrot)
        outs.append(F.attn(q_w, w_kc, w_vc, pos, None))
    want = torch.cat(outs)
    p_kc, p_vc, q_p, pos = dev(kc.view(np.int16)), dev(vc.view(np.int16)), dev(qg), dev(np.array([pos0], np.int32))
    F.attn_prep_append(q_p, dev(k), dev(v), qn, kn, p_kc, p_vc, pos, None, nrot)
    assert torch.equal(p_kc[:pos0 + T], w_kc[:pos0 + T]) and torch.equal(p_vc[:pos0 + T], w_vc[:pos0 + T])
    # both forms: sixteen rows per block on tcgen05.mma (this shape: eight query heads per KV head), twelve on mma.sync
    for mma_sync in (False, True):
        got = F.attn_prompt(q_p, p_kc, p_vc, pos, mma_sync=mma_sync)
        assert rel_err(got.cpu().numpy(), want.cpu().numpy()) < 2e-3, mma_sync
        if T <= 20:   # and against the oracle (a chain: no parents)
            ref = O.attn(q_p.cpu().numpy(), p_kc.cpu().numpy().view(np.uint16), p_vc.cpu().numpy().view(np.uint16), pos0, None)
            assert rel_err(got.cpu().numpy(), ref) < 2e-3, mma_sync


# ------------------------------------------------------------------------------------------------ DeltaNet
def _gdn_inputs(rng, T, nk, nv, hs):
    ch = (2 * nk + nv) * hs
    qkvz = rng.standard_normal((T, ch + nv * hs)).astype(np.float32)
    ab = rng.standard_normal((T, 2 * nv)).astype(np.float32)
    convw = (0.5 * rng.standard_normal((ch, 4))).astype(np.float32)
    dt = (0.1 * rng.standard_normal(nv)).astype(np.float32)
    a = (-np.exp(0.3 * rng.standard_normal(nv))).astype(np.float32)
    nw = (1 + 0.1 * rng.standard_normal(hs)).astype(np.float32)
    return ch, qkvz, ab, convw, dt, a, nw


@pytest.mark.parametrize("T,tree,nk,nv", [(1, False, 2, 4), (5, False, 16, 32), (6, True, 2, 4), (20, True, 4, 8)])
def test_gdn_core_matches_oracle(F, O, T, tree, nk, nv):
    hs, NS, cur = 128, T + 2, 3 % (T + 2)
    rng = np.random.default_rng(T * 10 + nv)
    ch, qkvz, ab, convw, dt, a, nw = _gdn_inputs(rng, T, nk, nv, hs)
    S = (0.1 * rng.standard_normal((NS, nv, hs, hs))).astype(np.float32)
    hist = rng.standard_normal((NS, 3, ch)).astype(np.float32)
    parent = [-1] + [int(rng.integers(0, t)) for t in range(1, T)] if tree else None
    d_S, d_hist = dev(S), dev(hist)
    y = F.gdn_core(dev(qkvz), dev(ab), d_hist, dev(convw), dev(dt), dev(a), dev(nw), d_S, dev(np.array([cur], np.int32)),
                   None if parent is None else dev(np.array(parent, np.int32)), nk, nv, hs)
    ref = O.gdn_core(qkvz, ab, hist, convw, dt, a, nw, S, cur, parent, nk, nv, hs)
    assert rel_err(y.cpu().numpy(), ref) < 2e-3      # the reference's own bar for two steps is 2e-3 (selftest.cu:257-302)
    assert rel_err(d_S.cpu().numpy(), S) < 1e-4
    assert np.array_equal(d_hist.cpu().numpy(), hist)           # histories are copies: bit-exact
    assert np.array_equal(d_S.cpu().numpy()[cur], S[cur])       # the starting slot is untouched


@pytest.mark.parametrize("T,NS", [(1, 4), (37, 9), (64, 33), (99, 33)])
def test_gdn_prompt_equals_chained_windows(F, O, T, NS):
    """The prompt form (conv / scan / norm in three launches, state in registers across all rows) against chained windows of
    NS - 1 rows of the window kernel, each kept whole: outputs, the final state and the final history."""
    nk, nv, hs, cur = 2, 4, 128, 2
    rng = np.random.default_rng(T + NS)
    ch, qkvz, ab, convw, dt, a, nw = _gdn_inputs(rng, T, nk, nv, hs)
    S0 = (0.1 * rng.standard_normal((NS, nv, hs, hs))).astype(np.float32)
    h0 = rng.standard_normal((NS, 3, ch)).astype(np.float32)
    args = (dev(convw), dev(dt), dev(a), dev(nw))
    Sw, Hw = dev(S0), dev(h0)
    ys, c, W = [], cur, NS - 1
    for t0 in range(0, T, W):
        nt = min(W, T - t0)
        ys.append(F.gdn_core(dev(qkvz[t0:t0 + nt]), dev(ab[t0:t0 + nt]), Hw, *args, Sw, dev(np.array([c], np.int32)), None, nk, nv, hs))
        c = (c + nt) % NS
    want = torch.cat(ys)
    Sp, Hp = dev(S0), dev(h0)
    got = F.gdn_prompt(dev(qkvz), dev(ab), Hp, *args, Sp, cur, nk, nv, hs)
    assert rel_err(got.cpu().numpy(), want.cpu().numpy()) < 1e-4
    if T <= 40:   # and against the row-by-row oracle over the whole chain at once
        So = np.concatenate([S0[cur:cur + 1], np.zeros((T + 1, nv, hs, hs), np.float32)])
        ho = np.concatenate([h0[cur:cur + 1], np.zeros((T + 1, 3, ch), np.float32)])
        ref = O.gdn_core(qkvz, ab, ho, convw, dt, a, nw, So, 0, None, nk, nv, hs)
        assert rel_err(got.cpu().numpy(), ref) < 2e-3
    out = (cur + T) % NS
    assert out == c
    assert rel_err(Sp[out].cpu().numpy(), Sw[out].cpu().numpy()) < 1e-4
    assert torch.equal(Hp[out], Hw[out])


def test_gdn_rollback_equals_running_only_the_kept_rows(F, O):
    # a 5-row chain cut back to 2 rows leaves the state a 2-row window leaves
    nk, nv, hs, T, NS = 2, 4, 128, 5, 6
    rng = np.random.default_rng(9)
    ch, qkvz, ab, convw, dt, a, nw = _gdn_inputs(rng, T, nk, nv, hs)
    S0 = (0.1 * rng.standard_normal((NS, nv, hs, hs))).astype(np.float32)
    h0 = rng.standard_normal((NS, 3, ch)).astype(np.float32)
    args = (dev(convw), dev(dt), dev(a), dev(nw))
    cur = dev(np.array([0], np.int32))
    S5, H5 = dev(S0), dev(h0)
    F.gdn_core(dev(qkvz), dev(ab), H5, *args[:4], S5, cur, None, nk, nv, hs)
    S2, H2 = dev(S0), dev(h0)
    F.gdn_core(dev(qkvz[:2]), dev(ab[:2]), H2, *args[:4], S2, cur, None, nk, nv, hs)
    assert torch.equal(S5[2], S2[2]) and torch.equal(H5[2], H2[2])   # slot 1 + 1 = state after row 1


# ------------------------------------------------------------------------------------------------ head
def test_argmax_and_top_tokens(F, O):
    rng = np.random.default_rng(31)
    T, V = 5, 151936
    logits = rng.standard_normal((T, V)).astype(np.float32)
    logits[1, 500] = logits[1, 70000] = 9.0          # a tie: the lower index wins
    logits[2, :] = 0.25                              # all equal
    logits[3, 10:90] = 7.0                           # more than 64 equal candidates
    bi, bv, err = F.argmax(dev(logits))
    ri, rv = O.argmax(logits)
    assert np.array_equal(bi.cpu().numpy(), ri) and np.array_equal(bv.cpu().numpy(), rv) and int(err.item()) == 0
    ov, oi = F.top_tokens(dev(logits))
    rv64, ri64 = O.top_tokens(logits)
    assert np.array_equal(oi.cpu().numpy(), ri64) and np.array_equal(ov.cpu().numpy(), rv64)
    logits[4, 123] = np.inf
    _, _, err = F.argmax(dev(logits))
    assert int(err.item()) == 16


# ------------------------------------------------------------------------------------------------ drafting, acceptance
def _edit_like_context(rng, n, vocab=5000):
    ctx = rng.integers(0, vocab, size=n).astype(np.int32)
    i = 300
    while i < n:
        if rng.random() < 0.6:
            ln = int(rng.integers(20, 200))
            s = int(rng.integers(0, i - ln)) if i - ln > 0 else 0
            ln = min(ln, n - i)
            ctx[i:i + ln] = ctx[s:s + ln]
            i += ln
        else:
            i += int(rng.integers(1, 40))
    return ctx


def test_lookup_matches_oracle_and_reference(F, O):
    rng = np.random.default_rng(2)
    ctx = _edit_like_context(rng, 32768)
    d_ctx = dev(ctx)
    hits = 0
    for n in list(rng.integers(4, 32768, size=60)) + [3, 4, 32768]:
        n = int(n)
        for lk in (15, 0, 5):
            for d1 in (-1, int(ctx[min(n, 32767)]), 7):
                want, wm = O.lookup(ctx[:n], lk, d1)
                got, gm = F.lookup_draft(d_ctx, dev(np.array([n], np.int32)), lk, dev(np.array([d1], np.int32)))
                assert got == list(want) and gm == wm
                hits += len(got) > 0
    assert hits > 10


def test_accept_greedy_tree(F, O):
    rng = np.random.default_rng(4)
    for _ in range(50):
        T = int(rng.integers(1, 21))
        parent = [-1] + [int(rng.integers(0, t)) for t in range(1, T)]
        tok = rng.integers(0, 6, size=T).astype(np.int32)
        best = rng.integers(0, 6, size=T).astype(np.int32)
        n, path, em = O.accept_greedy(tok, parent, best)
        gn, gpath, gem = F.accept_greedy(dev(tok), dev(np.array(parent, np.int32)), dev(best))
        assert (gn, gpath, gem) == (n, list(path), list(em))
    # chain with null parent
    tok = np.array([5, 1, 2, 3, 9], np.int32)
    best = np.array([1, 2, 3, 4, 0], np.int32)
    assert F.accept_greedy(dev(tok), None, dev(best)) == (4, [0, 1, 2, 3], [1, 2, 3, 4])


def test_accept_sample_counts_match_oracle(F, O):
    rng = np.random.default_rng(8)
    V, T = 4096, 5
    total = 0
    for it in range(40):
        logits = (rng.standard_normal((T, V)) * 3).astype(np.float32)
        cv, ci = O.top_tokens(logits)
        tok = rng.integers(0, V, size=T).astype(np.int32)
        for t in range(1, T):          # make most drafts likely ones
            tok[t] = ci[t - 1, int(rng.integers(0, 3))]
        for s in (O.Sampling(0.7, 1.0, 0.0, 0), O.Sampling(1.0, 0.9, 0.05, 40)):
            n, em = O.accept_sample(cv, ci, tok, s, seed=1234, seq=it, step=7)
            fs = F.Sampling(s.temperature, s.top_p, s.min_p, s.top_k)
            gn, _, gem = F.accept_sample(dev(cv), dev(ci), dev(tok), fs, 1234, it, dev(np.array([7], np.uint32).view(np.int32)))
            assert gn == n and gem == list(em)       # accepted counts and tokens: bit-exact
            total += n
    assert total > 80   # the cases do accept drafts


def test_philox_stream_matches_oracle(F, O):
    # known-answer vector of Philox4x32-10 (Random123 kat_vectors: zero counter and key)
    assert list(O.philox([0, 0, 0, 0], [0, 0])) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert list(O.philox([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2)) == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]


def test_cpp_consumer_of_the_header(F):
    """A C++ program compiled against include/fnx_b200.h and linked with the library calls fnx_dense and fnx_router_route on
    the GPU (tests/csrc/consumer.cpp): the header is what a consumer compiles, not only a list of names."""
    import pathlib
    import subprocess
    root = pathlib.Path(__file__).resolve().parent.parent
    pkg = next(p for p in root.iterdir() if p.is_dir() and (p / "libfnx_b200.so").exists())
    exe = root / "tests" / "csrc" / "consumer"
    cuda = pathlib.Path("/usr/local/cuda")
    cmd = ["g++", "-std=c++17", "-O1", "-I", str(root / "include"), "-I", str(cuda / "include"), str(root / "tests" / "csrc" / "consumer.cpp"), "-o", str(exe),
           "-L", str(pkg), "-lfnx_b200", "-L", str(cuda / "lib64"), "-lcudart", f"-Wl,-rpath,{pkg}", f"-Wl,-rpath,{cuda / 'lib64'}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    for rows, cols in ((256, 1024), (512, 2048)):
        r = subprocess.run([str(exe), str(rows), str(cols)], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0 and r.stdout.startswith("ok "), (r.returncode, r.stdout, r.stderr)


def test_logit_adjust_matches_oracle(F, O):
    """fnx_logit_adjust against the oracle's restatement, bit for bit: bias only, penalties only, both, windows shorter and longer
    than the context, a token in both lists, tokens outside the vocabulary (image cells) skipped."""
    rng = np.random.default_rng(5)
    V = 3000
    for T, n_ctx, last_n, rep, fr, pr, nb in [(1, 0, 8, 1.2, 0.1, 0.3, 0), (5, 200, 64, 1.3, 0.0, 0.0, 4), (8, 40, 4096, 0.9, 0.2, -0.5, 300), (3, 7000, 4096, 1.05, 0.01, 0.0, 1),
                                              (6, 10, 0, 1.0, 0.0, 0.0, 17), (4, 33, 1, 2.0, 1.0, 1.0, 2)]:
        logits = rng.standard_normal((T, V)).astype(np.float32) * 4
        ctx = rng.integers(0, 60, size=n_ctx).astype(np.int32)
        if n_ctx > 3:
            ctx[1] = V + 5            # not a vocabulary token
        tok = rng.integers(0, 60, size=T).astype(np.int32)
        bt = rng.choice(V, size=nb, replace=False).astype(np.int32)
        if nb:
            bt[0] = tok[0]
        bv = (rng.standard_normal(nb) * 3).astype(np.float32)
        want = O.logit_adjust(logits, ctx, tok, last_n, rep, fr, pr, list(zip(bt.tolist(), bv.tolist())))
        d = torch.from_numpy(logits).cuda()
        F.logit_adjust(d, torch.from_numpy(np.concatenate([ctx, np.zeros(1, np.int32)])).cuda(), torch.tensor([n_ctx], dtype=torch.int32, device="cuda"),
                       torch.from_numpy(tok).cuda(), last_n, rep, fr, pr, torch.from_numpy(bt).cuda() if nb else None, torch.from_numpy(bv).cuda() if nb else None)
        assert np.array_equal(d.cpu().numpy().view(np.uint32), want.view(np.uint32)), (T, n_ctx, last_n)
