"""GPU tests of the window scheduler (Engine::verify / commit / draft over the C ABI) on a reduced model, against the
same model run through the CPU oracle, plus the size-independent properties the reference's own `spec` test uses:
speculative output equals plain greedy output, and a cut-back window leaves the state of a window of the kept rows."""
import numpy as np
import pytest

from helpers import OracleModel, rel_err

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def small_cfg(F, **over):
    # every kernel path at a different shape from the benchmark's: hidden 1024 (4 blocks per row), ffn 256
    d = dict(n_layer=4, hidden=1024, n_expert=32, top_k=4, ffn=256, n_q_head=8, n_kv_head=1, head_dim=256, n_rot=64, gdn_k_head=2,
             gdn_v_head=4, gdn_head_dim=128, vocab=2048, max_ctx=512, max_rows=8, attn_every=4)
    d.update(over)
    return F.flash_next_config(**d)


@pytest.fixture(scope="module")
def model(F, O):
    cfg = small_cfg(F)
    eng = F.Engine(cfg)
    eng.init_synthetic(seed=0, sigma=0.02)
    om = OracleModel(F, O, eng, cfg)
    yield cfg, eng, om
    eng.close()


def _routing_margin_ok(om, K, tol=2e-4):
    """True when every row's K-th and (K+1)-th router logits are further apart than the kernels' rounding."""
    for topi, logits in om.routing:
        for t in range(topi.shape[0]):
            l = np.sort(logits[t, :-1])[::-1]
            if l[K - 1] - l[K] < tol * max(1.0, abs(l[0])):
                return False
    return True


def test_verify_commit_draft_match_oracle(F, O, model):
    cfg, eng, om = model
    rng = np.random.default_rng(0)
    eng.reset()
    # 1) a prompt of 19 tokens through chained windows
    prompt = rng.integers(0, cfg.vocab, size=19).tolist()
    eng.prefill(prompt)
    for i in range(0, len(prompt), cfg.max_rows):
        w = prompt[i:i + cfg.max_rows]
        om.verify(w, None)
        om.commit(list(range(len(w))))
    assert eng.pos() == om.pos == 19
    # 2) a chain window of 5 rows
    toks = rng.integers(0, cfg.vocab, size=5).tolist()
    n, path, em = eng.verify(toks)
    on, opath, oem = om.verify(toks, None)
    R = eng.tensor("buf.R", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.hidden)[:5]
    logits = eng.tensor("buf.logits", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.vocab)[:5]
    topi = eng.tensor("buf.topi", torch.int32).cpu().numpy().reshape(cfg.max_rows, cfg.top_k)[:5]
    assert _routing_margin_ok(om, cfg.top_k), "pick another seed: a routing near-tie makes the comparison meaningless"
    assert rel_err(R, om.R) < 1e-2 and rel_err(logits, om.logits) < 1e-2           # the target's bar
    assert rel_err(R, om.R) < 2e-3                                                   # what the kernels hold
    assert np.array_equal(topi, om.routing[-1][0])                                   # last layer's routing, bit-exact
    assert (n, path, em) == (on, list(opath), list(oem))
    # 3) keep what greedy accepted, draft 3 tokens with the MTP layer
    eng.commit(path)
    om.commit(list(opath))
    d = eng.draft(3)
    od = om.draft(list(oem), 3)
    assert d == od
    # 4) a tree window: the accepted token as root, two branches
    root = em[-1]
    toks = [root, d[0], d[1], int(rng.integers(0, cfg.vocab)), d[2], int(rng.integers(0, cfg.vocab))]
    par = [-1, 0, 1, 0, 2, 3]
    r1 = eng.verify(toks, par)
    r2 = om.verify(toks, par)
    R = eng.tensor("buf.R", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.hidden)[:6]
    assert rel_err(R, om.R) < 2e-3
    assert r1 == (r2[0], list(r2[1]), list(r2[2]))
    # keep a path that is not a prefix of the rows, to exercise the cache compaction and the state ring
    keep = [0, 3, 5]
    eng.commit(keep)
    om.commit(keep)
    toks = rng.integers(0, cfg.vocab, size=3).tolist()
    r1 = eng.verify(toks)
    r2 = om.verify(toks, None)
    R = eng.tensor("buf.R", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.hidden)[:3]
    assert rel_err(R, om.R) < 2e-3
    assert r1 == (r2[0], list(r2[1]), list(r2[2]))


def test_drafts_over_a_draft_vocabulary_match_oracle(F, O):
    """The draft layer with its own head over a draft vocabulary (Mtp::vocab of the reference: head row -> token id): the
    chained drafts are the oracle's, they are ids of that vocabulary, and the batched chain gives the same tokens."""
    cfg = small_cfg(F, draft_vocab=512, n_seq=2)
    eng = F.Engine(cfg)
    try:
        eng.init_synthetic(seed=3, sigma=0.02)
        om = OracleModel(F, O, eng, cfg)
        assert om.dvocab.shape == (512,) and np.all(np.diff(om.dvocab) > 0) and om.dvocab[-1] < cfg.vocab
        rng = np.random.default_rng(5)
        eng.reset()
        toks = rng.integers(0, cfg.vocab, size=5).tolist()
        n, path, em = eng.verify(toks)
        on, opath, oem = om.verify(toks, None)
        assert (n, path, em) == (on, list(opath), list(oem))
        eng.commit(path)
        om.commit(list(opath))
        d = eng.draft(3)
        assert d == om.draft(list(oem), 3)
        assert all(t in set(om.dvocab.tolist()) for t in d)
        # the same window on a second sequence through the batched lanes
        res = eng.verify_lanes([1], [toks])
        assert res[0] == (n, path, em)
        eng.commit_lanes([1], [len(path)])
        assert eng.draft_lanes([1], 3) == [d]
    finally:
        eng.close()


def test_prompt_pass_matches_the_window_path_and_the_oracle(F, O, model):
    """A 75-token prompt through fnx_engine_prompt (tensor-core projections and experts, chained DeltaNet windows): positions,
    context and emitted token equal the window path's (itself checked against the oracle above), the following window agrees
    with it to the parity tolerance (activations are f16 in the prompt pass), and drafts and lookup still work."""
    cfg, eng, om = model
    rng = np.random.default_rng(11)
    prompt = rng.integers(0, cfg.vocab, size=75).tolist()
    eng.reset()
    eng.prefill(prompt)
    pos_w = eng.pos()
    toks = rng.integers(0, cfg.vocab, size=5).tolist()
    want = eng.verify(toks)
    R_w = eng.tensor("buf.R", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.hidden)[:5].copy()
    lg_w = eng.tensor("buf.logits", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.vocab)[:5].copy()
    ctx_w = eng.tensor("seq.ctx", torch.int32).cpu().numpy()[:pos_w + 1].copy()
    eng.reset()
    eng.prompt(prompt)
    assert eng.pos() == pos_w == 75 and eng.error_bits() == 0
    assert np.array_equal(eng.tensor("seq.ctx", torch.int32).cpu().numpy()[:pos_w], ctx_w[:pos_w])
    got = eng.verify(toks)
    R_p = eng.tensor("buf.R", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.hidden)[:5]
    lg_p = eng.tensor("buf.logits", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.vocab)[:5]
    assert rel_err(R_p, R_w) < 5e-3 and rel_err(lg_p, lg_w) < 5e-3
    assert got[0] >= 1 and len(got[1]) == got[0]
    eng.commit(got[1])
    assert len(eng.draft(2)) == 2
    # a prompt of one token, and one that ends exactly on a window boundary
    for n in (1, 2 * cfg.max_rows + 1):
        eng.reset()
        eng.prompt(prompt[:n])
        assert eng.pos() == n and eng.error_bits() == 0


def test_saved_state_brings_a_sequence_back_bit_for_bit(F):
    """save_state / load_state: after a prompt, two more windows and a load, the same window gives the same bits again - with the
    cache rows in the image (also into another sequence) and without them (a rewind of the same sequence); a checkpoint
    without K/V is refused for a sequence that does not continue it, and neither call may fall between verify and commit."""
    cfg = small_cfg(F, n_seq=2)
    eng = F.Engine(cfg)
    try:
        eng.init_synthetic(seed=5, sigma=0.02)
        rng = np.random.default_rng(21)
        prompt = rng.integers(0, cfg.vocab, size=21).tolist()
        wins = [rng.integers(0, cfg.vocab, size=5).tolist() for _ in range(3)]

        def window(seq, toks):
            r = eng.verify(toks, None, seq)
            lg = eng.tensor("buf.logits", torch.float32).cpu().reshape(cfg.max_rows, cfg.vocab)[:len(toks)].clone()
            return r, lg

        eng.reset(0)
        eng.prefill(prompt, 0)
        full = eng.save_state(0, kv=True)
        light = eng.save_state(0, kv=False)
        assert len(light) < len(full)
        r0, lg0 = window(0, wins[0])
        with pytest.raises(F.FnxError):
            eng.save_state(0)                      # a window is pending
        eng.commit(r0[1], 0)
        r1, _ = window(0, wins[1])
        eng.commit(r1[1], 0)
        assert eng.pos(0) > 21
        # a rewind without K/V: the engine still holds the rows
        eng.load_state(light, 0)
        assert eng.pos(0) == 21
        ra, lga = window(0, wins[0])
        assert ra == r0 and torch.equal(lga, lg0)
        eng.commit(ra[1], 0)
        # the full image into the other sequence
        eng.load_state(full, 1)
        assert eng.pos(1) == 21
        rb, lgb = window(1, wins[0])
        assert rb == r0 and torch.equal(lgb, lg0)
        eng.commit(rb[1], 1)
        assert len(eng.draft(2, 1)) == 2
        # sequence 1 after a reset does not continue the checkpoint: without K/V it is refused, with K/V it loads
        eng.reset(1)
        eng.prefill(wins[2], 1)
        with pytest.raises(F.FnxError):
            eng.load_state(light, 1)
        eng.load_state(full, 1)
        rc, lgc = window(1, wins[0])
        assert rc == r0 and torch.equal(lgc, lg0)
        eng.commit(rc[1], 1)
    finally:
        eng.close()


def test_full_size_layers_match_oracle(F, O):
    """The benchmark model's own dimensions (hidden 2048, 512 experts top-10 of width 512, 16/2 attention heads of 256, 16/32
    DeltaNet heads of 128, vocabulary 151,936), four layers of it (three DeltaNet, one attention): a prompt, a 5-row chain window
    (the benchmark's window: ~50 expert jobs per layer, walked in several passes per block, expert strides of 1.35 MB) and a
    tree window, against the oracle: the last layer's routing indices bit-exact (an earlier layer's mismatch would show in the
    hidden states), hidden states and logits within the kernels' 2e-3 (the target asks 1e-2), accepted path and tokens equal."""
    cfg = F.flash_next_config(n_layer=4, max_ctx=256, max_rows=8)
    eng = F.Engine(cfg)
    try:
        eng.init_synthetic(seed=0, sigma=0.02)
        om = OracleModel(F, O, eng, cfg, with_mtp=False)
        rng = np.random.default_rng(5)
        prompt = rng.integers(0, cfg.vocab, size=21).tolist()
        eng.reset()
        eng.prefill(prompt)
        for i in range(0, len(prompt), cfg.max_rows):
            w = prompt[i:i + cfg.max_rows]
            om.verify(w, None)
            om.commit(list(range(len(w))))
        for T, par in ((5, None), (7, [-1, 0, 1, 0, 3, 3, 1])):
            # top-K is discontinuous: among 512 experts some window has a K-th / (K+1)-th logit pair closer than the kernels'
            # rounding; take the first seeded window without one (a window changes no committed state, so trying one is free)
            for _ in range(8):
                toks = rng.integers(0, cfg.vocab, size=T).tolist()
                want = om.verify(toks, par)
                if _routing_margin_ok(om, cfg.top_k):
                    break
            else:
                raise AssertionError("eight windows in a row with a routing near-tie")
            got = eng.verify(toks, par)
            R = eng.tensor("buf.R", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.hidden)[:T]
            logits = eng.tensor("buf.logits", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.vocab)[:T]
            topi = eng.tensor("buf.topi", torch.int32).cpu().numpy().reshape(cfg.max_rows, cfg.top_k)[:T]
            assert np.array_equal(topi, om.routing[-1][0])
            assert rel_err(R, om.R) < 2e-3 and rel_err(logits, om.logits) < 2e-3
            assert got == (want[0], list(want[1]), list(want[2]))
            assert eng.error_bits() == 0
            eng.commit(got[1])
            om.commit(list(want[1]))
    finally:
        eng.close()


def _greedy_plain(eng, prompt, steps):
    eng.reset()
    eng.prefill(prompt[:-1])
    x, out = prompt[-1], []
    for _ in range(steps):
        n, path, em = eng.verify([x])
        eng.commit([0])
        x = em[0]
        out.append(x)
    return out


def test_speculative_output_equals_plain_greedy(F, model):
    """K perfect drafts, and windows with a corrupted draft: the emitted text must be the plain greedy text (the
    reference's `spec` mode, engine/tools/fnx_run.cpp:8-9)."""
    cfg, eng, _ = model
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, cfg.vocab, size=12).tolist()
    want = _greedy_plain(eng, prompt, 24)
    eng.reset()
    eng.prefill(prompt[:-1])
    x, out, i = prompt[-1], [], 0
    while len(out) < 24:
        k = min(4, 24 - len(out) - 1)
        drafts = list(want[len(out):len(out) + k])
        if k and i % 3 == 1:
            j = int(rng.integers(0, k))
            drafts[j] = (drafts[j] + 1) % cfg.vocab        # one wrong draft: the window is cut back there
        n, path, em = eng.verify([x] + drafts)
        assert path == list(range(n))
        if not (k and i % 3 == 1):
            assert n == k + 1
        eng.commit(path)
        out += em
        x = em[-1]
        i += 1
    assert out[:24] == want


def test_tree_verify_equals_chain_verify_of_the_accepted_path(F, model):
    cfg, eng, _ = model
    rng = np.random.default_rng(6)
    prompt = rng.integers(0, cfg.vocab, size=9).tolist()
    want = _greedy_plain(eng, prompt, 6)
    eng.reset()
    eng.prefill(prompt[:-1])
    # root, a wrong branch first, then the right chain hanging off the root as a second branch
    wrong = [(want[0] + 7) % cfg.vocab, (want[1] + 7) % cfg.vocab]
    toks = [prompt[-1], wrong[0], wrong[1], want[0], want[1], want[2]]
    par = [-1, 0, 1, 0, 3, 4]
    n, path, em = eng.verify(toks, par)
    assert path == [0, 3, 4, 5] and em == want[:4]
    eng.commit(path)
    n, path, em = eng.verify([em[-1]])
    assert em[0] == want[4]


def test_engine_rejects_bad_calls(F, model):
    cfg, eng, _ = model
    eng.reset()
    with pytest.raises(F.FnxError):
        eng.verify([1] * (cfg.max_rows + 1))
    with pytest.raises(F.FnxError):
        eng.verify([cfg.vocab])
    with pytest.raises(F.FnxError):
        eng.verify([1, 2], [-1, 1])       # a parent must be an earlier row
    with pytest.raises(F.FnxError):
        eng.commit([0])                   # nothing verified
    eng.verify([1, 2, 3])
    with pytest.raises(F.FnxError):
        eng.commit([0, 2, 1])
    eng.commit([0])


def test_lookup_branch_and_draft_chain_in_one_tree_window(F, O, model):
    """The second configuration's window: an MTP-style chain and a prompt-lookup branch share the root of one tree
    window; the kept path is the branch that continues the greedy text, whichever it is."""
    cfg, eng, _ = model
    rng = np.random.default_rng(12)
    span = rng.integers(0, cfg.vocab, size=10).tolist()
    prompt = rng.integers(0, cfg.vocab, size=6).tolist() + span + rng.integers(0, cfg.vocab, size=5).tolist() + span[:4]
    want = _greedy_plain(eng, prompt, 8)
    eng.reset()
    eng.prefill(prompt[:-1])
    # the device drafter over the engine's own context equals the reference's host drafter on the same tokens
    lk = eng.lookup(3, root=prompt[-1])
    assert lk == list(O.lookup(np.array(prompt, np.int32), 3, -1)[0]) and lk == span[4:7]
    chain = [want[0], want[1], (want[2] + 1) % cfg.vocab]         # a draft chain with one wrong token
    toks = [prompt[-1]] + chain + lk
    par = [-1, 0, 1, 2] + [0] + list(range(4, 4 + len(lk) - 1))
    n, path, em = eng.verify(toks, par)
    # greedy acceptance follows the branch whose tokens match: the chain's first two (the lookup branch is the copied span,
    # not the model's greedy text, unless they coincide)
    assert em[:n] == want[:n] and n >= 3 and path[:3] == [0, 1, 2]
    eng.commit(path)
    n2, _, em2 = eng.verify([em[-1]])
    assert em2[0] == want[n]


def test_engine_sampling_windows_follow_the_oracle_rule(F, O, model):
    """Stochastic acceptance inside the engine (the fourth configuration's rule): accepted counts and emitted tokens equal
    the oracle's rule applied to the engine's own logits, window after window (Philox step = window index)."""
    cfg, eng, _ = model
    rng = np.random.default_rng(13)
    prompt = rng.integers(0, cfg.vocab, size=10).tolist()
    s = F.Sampling(0.7, 0.95, 0.02, 40)
    eng.reset()
    eng.set_sampling(s, seed=77)
    try:
        eng.prefill(prompt[:-1])
        # prefill windows are sampled windows too: the Philox step counts them
        step0 = (len(prompt) - 1 + cfg.max_rows - 1) // cfg.max_rows
        x, accepted = prompt[-1], 0
        for w in range(6):
            drafts = eng.draft(3)
            toks = [x] + drafts
            n, path, em = eng.verify(toks)
            logits = eng.tensor("buf.logits", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.vocab)[:len(toks)]
            cv, ci = O.top_tokens(logits)
            on, oem = O.accept_sample(cv, ci, np.array(toks, np.int32), O.Sampling(s.temperature, s.top_p, s.min_p, s.top_k), seed=77, seq=0,
                                      step=step0 + w)
            assert (n, em) == (on, list(oem)) and path == list(range(n))
            accepted += n - 1
            eng.commit(path)
            x = em[-1]
        with pytest.raises(F.FnxError):
            eng.verify([x, 1, 2], [-1, 0, 0])          # the sampling rule is defined on chains
    finally:
        eng.set_sampling(None)


def test_a_row_gives_the_same_bits_alone_and_among_drafts(F, model):
    """Window invariance: a row's logits do not depend on the window it is verified in (attention partials are cut at
    absolute positions, expert K-sums are accumulated in double, everything else is per row).  This is what makes
    speculative output equal plain greedy output for any number of steps, not only up to the first near-tie."""
    cfg, eng, _ = model
    rng = np.random.default_rng(14)
    prompt = rng.integers(0, cfg.vocab, size=70).tolist()
    toks = rng.integers(0, cfg.vocab, size=5).tolist()
    eng.reset()
    eng.prefill(prompt)
    eng.verify(toks)
    together = eng.tensor("buf.logits", torch.float32).view(cfg.max_rows, cfg.vocab)[:5].clone()
    eng.reset()
    eng.prefill(prompt)
    for i, t in enumerate(toks):
        eng.verify([t])
        eng.commit([0])
        alone = eng.tensor("buf.logits", torch.float32).view(cfg.max_rows, cfg.vocab)[0]
        assert torch.equal(alone, together[i]), f"row {i}"


@pytest.mark.parametrize("sampling", [False, True])
def test_batched_lanes_equal_single_sequence_windows(F, sampling):
    """Three sequences of different lengths in one window (Engine::verify_rows): every lane's accepted tokens, hidden rows and
    logits are bit-identical to the same rows run through the single-sequence window of that sequence alone, for the greedy
    and for the sampling rule (each sequence draws its own Philox stream); so are the MTP drafts of the batched chain, and
    so is a second window after the lanes kept different numbers of rows."""
    cfg = small_cfg(F, n_seq=3, max_rows=16)
    eng = F.Engine(cfg)
    try:
        eng.init_synthetic(seed=0, sigma=0.02)
        rng = np.random.default_rng(21)
        prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (9, 14, 6)]
        rounds = [[rng.integers(0, cfg.vocab, size=4).tolist() for _ in range(3)] for _ in range(2)]
        seqs = [0, 1, 2]
        samp = F.Sampling(0.8, 0.95, 0.0, 40)

        def begin():
            eng.set_sampling(samp if sampling else None, seed=77)
            for s in seqs:
                eng.reset(s)
                eng.prefill(prompts[s], s)

        def rows_of(name, width, lo, n):
            return eng.tensor(name, torch.float32).cpu().numpy().reshape(cfg.max_rows, width)[lo:lo + n].copy()

        # ---- every sequence alone
        begin()
        alone = {s: [] for s in seqs}
        for s in seqs:
            for r in range(2):
                res = eng.verify(rounds[r][s], None, s)
                R, lg = rows_of("buf.R", cfg.hidden, 0, 4), rows_of("buf.logits", cfg.vocab, 0, 4)
                eng.commit(res[1], s)
                d = eng.draft(2, s)
                alone[s].append((res, R, lg, d))
        # ---- the same windows as lanes
        begin()
        for r in range(2):
            got = eng.verify_lanes(seqs, [rounds[r][s] for s in seqs])
            for j, s in enumerate(seqs):
                res, R, lg, d = alone[s][r]
                assert got[j] == res, (r, s, got[j], res)
                assert np.array_equal(rows_of("buf.R", cfg.hidden, 4 * j, 4), R)
                assert np.array_equal(rows_of("buf.logits", cfg.vocab, 4 * j, 4), lg)
            eng.commit_lanes(seqs, [g[0] for g in got])
            drafts = eng.draft_lanes(seqs, 2)
            for j, s in enumerate(seqs):
                assert drafts[j] == alone[s][r][3], (r, s, drafts[j], alone[s][r][3])
            assert eng.error_bits() == 0
        for s in seqs:
            assert eng.pos(s) == len(prompts[s]) + sum(alone[s][r][0][0] for r in range(2))
    finally:
        eng.set_sampling(None, 0)
        eng.close()


def test_lanes_of_different_lengths_equal_single_sequence_windows(F):
    """A planner's window: lanes of 5, 2 and 3 rows (fnx_engine_verify_lanes_rows).  Every lane's result and logits are
    bit-identical to the same rows through that sequence's own window, and so are the drafts after the commit."""
    cfg = small_cfg(F, n_seq=3, max_rows=16)
    eng = F.Engine(cfg)
    try:
        eng.init_synthetic(seed=0, sigma=0.02)
        rng = np.random.default_rng(33)
        prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (7, 12, 5)]
        wins = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (5, 2, 3)]
        seqs = [0, 1, 2]

        def begin():
            for s in seqs:
                eng.reset(s)
                eng.prefill(prompts[s], s)

        begin()
        alone = []
        for s in seqs:
            res = eng.verify(wins[s], None, s)
            lg = eng.tensor("buf.logits", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.vocab)[:len(wins[s])].copy()
            eng.commit(res[1], s)
            alone.append((res, lg, eng.draft(2, s)))
        begin()
        got = eng.verify_lanes_rows(seqs, wins)
        lg = eng.tensor("buf.logits", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.vocab)
        r0 = 0
        for j, s in enumerate(seqs):
            assert got[j] == alone[s][0]
            assert np.array_equal(lg[r0:r0 + len(wins[s])], alone[s][1])
            r0 += len(wins[s])
        with pytest.raises(F.FnxError):
            eng.commit_lanes(seqs, [5, 3, 3])          # lane 1 has two rows
        eng.commit_lanes(seqs, [g[0] for g in got])
        drafts = eng.draft_lanes(seqs, 2)
        assert drafts == [a[2] for a in alone] and eng.error_bits() == 0
    finally:
        eng.close()


def test_a_missing_peer_times_out_and_leaves_the_context_usable(F):
    """An expert-parallel rank whose peer never answers: the exchange's bounded wait runs out (a flag that nothing sets), the
    window reports FNX_ERR_TIMEOUT through the err word instead of hanging, and the same engine keeps answering calls."""
    cfg = small_cfg(F, ep_rank=0, ep_size=2)
    eng = F.Engine(cfg)
    try:
        eng.init_synthetic(seed=0, sigma=0.02)
        F.check(F.lib().fnx_engine_ep_open_loopback(eng._h))
        F.check(F.lib().fnx_engine_set_wait_limit(eng._h, 20000))
        with pytest.raises(F.FnxError) as ei:
            eng.verify([1, 2, 3])
        assert "0x1" in str(ei.value) or "bits" in str(ei.value)
        assert eng.error_bits() & 1
        # the context is intact: the next call runs (and times out again, quickly: one short wait per window)
        with pytest.raises(F.FnxError):
            eng.verify([4, 5])
        assert eng.pos() == 0
    finally:
        eng.close()


def _weight_names(eng_cfg):
    names = ["out_norm", "head", "embed", "mtp.e_norm", "mtp.h_norm", "mtp.out_norm", "mtp.fc_emb", "mtp.fc_hid"]
    for l in list(range(eng_cfg.n_layer)) + ["mtp"]:
        attn = l == "mtp" or (l + 1) % eng_cfg.attn_every == 0
        pre = "mtp." if l == "mtp" else f"l{l}."
        names += [pre + n for n in ("norm1", "norm2", "w_in", "w_out", "router", "experts_gu", "experts_dn", "shared_gu", "shared_dn")]
        names += [pre + n for n in (("q_norm", "k_norm") if attn else ("conv_w", "dt", "a", "g_norm"))]
    if eng_cfg.draft_vocab:
        names += ["mtp.head", "mtp.vocab"]
    return names


def test_gguf_load_restores_every_weight_bit(F, tmp_path):
    """An engine's weights written to a GGUF file under llama.cpp's names (gguf-py's writer) and loaded into a second engine:
    every weight tensor holds the same bytes, nothing had to be quantised, and both engines emit the same tokens.  An
    expert-parallel rank loads its own slice of the stacked expert tensors."""
    from gguf_files import model_meta, tiny_model_tensors, write_gguf
    cfg = small_cfg(F, draft_vocab=512)
    a = F.Engine(cfg)
    a.init_synthetic(seed=5, sigma=0.02)
    # vectors that the synthetic model leaves at 1: make them distinct so that a swapped name shows
    g0 = torch.Generator(device="cuda").manual_seed(1)
    for n in _weight_names(cfg):
        if n.endswith(("norm1", "norm2", "q_norm", "k_norm", "g_norm", "e_norm", "h_norm", "out_norm")):
            t = a.tensor(n, torch.float32)
            t.copy_(1.0 + 0.1 * torch.randn(t.shape, device="cuda", generator=g0))
    path = tmp_path / "tiny.gguf"
    write_gguf(path, model_meta(cfg), tiny_model_tensors(F, a, cfg))
    g = F.Gguf(path)
    cfg_b = g.model_config(max_ctx=cfg.max_ctx, max_rows=cfg.max_rows)
    b = F.Engine(cfg_b)
    assert b.load_gguf(g) == 0
    tile_rows = 16 * (16 // (cfg.hidden // 256))

    def in_rows(n):   # rows of an input projection that the file holds (the engine pads them to whole tiles; the padding stays zero)
        attn = n.startswith("mtp.") or (int(n[1:n.index(".")]) + 1) % cfg.attn_every == 0
        used = (cfg.n_q_head * 2 + 2 * cfg.n_kv_head) * cfg.head_dim if attn else (2 * cfg.gdn_k_head + 2 * cfg.gdn_v_head) * cfg.gdn_head_dim + 2 * cfg.gdn_v_head
        return used, (used + tile_rows - 1) // tile_rows * tile_rows

    def same(x, y, n):
        ta, tb = x.tensor(n, torch.uint8), y.tensor(n, torch.uint8)
        if not n.endswith("w_in"):
            return ta.shape == tb.shape and torch.equal(ta, tb)
        used, rows = in_rows(n)
        ga = F.iq3s_untile(ta, rows, cfg.hidden).view(rows, -1)
        gb = F.iq3s_untile(tb, rows, cfg.hidden).view(rows, -1)
        return torch.equal(ga[:used], gb[:used]) and int(gb[used:].abs().max() if rows > used else 0) == 0

    for n in _weight_names(cfg):
        assert same(a, b, n), n
    toks = np.random.default_rng(3).integers(0, cfg.vocab, size=7).tolist()
    for e in (a, b):
        e.reset()
        e.prefill(toks[:4])
    ra, rb = a.verify(toks[4:]), b.verify(toks[4:])
    assert ra == rb
    a.commit(ra[1]); b.commit(rb[1])
    assert a.draft(3) == b.draft(3)
    # rank 1 of 2: experts [16, 32) of the stacked tensors
    cfg_c = g.model_config(max_ctx=cfg.max_ctx, max_rows=cfg.max_rows, ep_rank=1, ep_size=2)
    c = F.Engine(cfg_c)
    assert c.load_gguf(g) == 0
    for n in ("l0.experts_gu", "l3.experts_dn", "mtp.experts_gu"):
        ta, tc = a.tensor(n, torch.uint8), c.tensor(n, torch.uint8)
        assert ta.numel() == 2 * tc.numel() and torch.equal(ta[tc.numel():], tc), n
    assert torch.equal(a.tensor("l1.router", torch.uint8), c.tensor("l1.router", torch.uint8))
    c.close()
    b.close()
    g.close()
    # the same model with some matrices in other formats: they are quantised on the way in (counted), the rest stays bit-equal,
    # and an architecture mismatch is refused
    from gguf import GGMLQuantizationType as QT
    from gguf.quants import dequantize, quantize
    t = tiny_model_tensors(F, a, cfg)
    H = cfg.hidden
    wo = dequantize(t["blk.3.attn_output.weight"][0], QT.IQ3_S).reshape(H, -1)
    t["blk.3.attn_output.weight"] = wo.astype(np.float16)
    al = dequantize(t["blk.0.ssm_alpha.weight"][0], QT.IQ3_S).reshape(-1, H)
    t["blk.0.ssm_alpha.weight"] = al.astype(np.float32)
    sd = dequantize(t["blk.1.ffn_down_shexp.weight"][0], QT.IQ3_S).reshape(H, -1)
    t["blk.1.ffn_down_shexp.weight"] = (quantize(sd, QT.Q8_0), QT.Q8_0)
    path2 = tmp_path / "mixed.gguf"
    write_gguf(path2, model_meta(cfg), t)
    g = F.Gguf(path2)
    b = F.Engine(g.model_config(max_ctx=cfg.max_ctx, max_rows=cfg.max_rows))
    assert b.load_gguf(g) == 3
    assert same(a, b, "l3.w_in") and same(a, b, "l0.w_out")
    # weights that IQ3_S holds exactly come back as the same values (f16 holds them exactly too; Q8_0 to its own rounding)
    wa = F.iq3s_dequant_tiles(a.tensor("l3.w_out", torch.uint8), H, wo.shape[1]).cpu().numpy()
    wb = F.iq3s_dequant_tiles(b.tensor("l3.w_out", torch.uint8), H, wo.shape[1]).cpu().numpy()
    assert np.linalg.norm(wb - wa) / np.linalg.norm(wa) < 0.1
    wrong = F.Engine(small_cfg(F, draft_vocab=512, n_layer=8))
    with pytest.raises(F.FnxError, match="architecture"):
        wrong.load_gguf(g)
    wrong.close()
    b.close()
    g.close()
    a.close()


class _Serve:
    """fnx_serve as a child process, spoken to a line at a time"""

    def __init__(self, *args):
        import pathlib
        import subprocess
        exe = pathlib.Path(__file__).resolve().parents[1] / "qwen3.8-flash-next-2x-p100_b200" / "fnx_serve"
        self.p = subprocess.Popen([str(exe), "--serve", *map(str, args)], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)

    def line(self):
        l = self.p.stdout.readline()
        assert l, "fnx_serve closed its output"
        return l.rstrip("\n")

    def send(self, *lines):
        self.p.stdin.write("".join(l + "\n" for l in lines))
        self.p.stdin.flush()

    def reply(self):
        """the lines of one request's answer: (PP lines, RESUME count, tokens, DONE fields) or the ERR line"""
        pp, toks, resume = [], [], None
        while True:
            l = self.line()
            w = l.split()
            if w[0] == "ERR":
                return l
            if w[0] == "PP":
                pp.append((int(w[1]), int(w[2])))
            elif w[0] == "RESUME":
                resume = int(w[1])
            elif w[0] == "T":
                toks.append(int(w[1]))
            elif w[0] == "DONE":
                return pp, resume, toks, w[1:]

    def quit(self):
        self.send("QUIT")
        return self.p.wait(timeout=60)


def test_serve_process_speaks_the_line_protocol(F, tmp_path):
    """fnx_serve on a small model file: a greedy request's tokens are the plain greedy tokens of the same engine calls made from
    Python (speculative windows change nothing), a prompt that goes on from the last one reuses it, seeded sampling repeats,
    STOP cancels, bad lines answer ERR and the process carries on."""
    from gguf_files import model_meta, tiny_model_tensors, write_gguf
    cfg = small_cfg(F, max_ctx=1024)
    a = F.Engine(cfg)
    a.init_synthetic(seed=9, sigma=0.02)
    path = tmp_path / "tiny.gguf"
    meta = model_meta(cfg)
    write_gguf(path, meta, tiny_model_tensors(F, a, cfg))
    rng = np.random.default_rng(21)
    prompt = rng.integers(0, cfg.vocab, size=40).tolist()

    def plain(eng, prompt, n_new, fresh=True):   # one-row greedy windows
        if fresh:
            eng.reset()
        if len(prompt) > 1:
            eng.prompt(prompt[:-1])
        x, out = prompt[-1], []
        for _ in range(n_new):
            n, path_, em = eng.verify([x])
            eng.commit([0])
            x = em[0]
            out.append(x)
        return out

    want = plain(a, prompt, 24)
    s = _Serve("--native", path, "--max-context", 1024, "--spec", 3, "--lookup", 6, "--prompt-chunk", 4096)
    assert s.line().startswith("INFO engine=fnx_b200 version=")
    assert s.line() == "READY 1024 stop"
    csv = lambda ids: ",".join(map(str, ids))
    s.send(f"GEN 24 {csv(prompt)}")
    pp, resume, toks, done = s.reply()
    assert pp == [(39, 39)] and resume == 0
    assert toks == want
    assert done[0] == "24" and done[1] == "40" and done[4] == "length" and int(done[6]) >= int(done[5]) >= 0 and done[7] == "0"
    # the conversation goes on: the engine holds the prompt and all but the last generated token
    more = prompt + want + rng.integers(0, cfg.vocab, size=9).tolist()
    s.send(f"GEN 10 {csv(more)}")
    pp, resume, toks2, done = s.reply()
    assert resume == len(prompt) + len(want) - 1 and pp == [(len(more) - 1, len(more) - 1)] and done[7] == str(resume)
    # the same from Python: the engine `a` holds prompt + want[:-1] too (its last window's token is not kept yet)
    a.prompt(more[len(prompt) + len(want) - 1:-1])
    x, want2 = more[-1], []
    for _ in range(10):
        n, path_, em = a.verify([x])
        a.commit([0])
        x = em[0]
        want2.append(x)
    assert toks2 == want2
    # a prompt that does not go on from the engine's tokens starts over; chunks of the read are reported
    s.send("GEN 3 " + csv(prompt[:30]))
    pp, resume, toks3, done = s.reply()
    assert resume == 0 and pp == [(29, 29)] and toks3 == plain(a, prompt[:30], 3)
    # seeded sampling repeats itself, whatever ran in between
    s.send(f"GEN 12 temperature=0.9 top_k=20 seed=77 {csv(prompt[:20])}")
    r1 = s.reply()
    s.send(f"GEN 5 {csv(prompt[:12])}")
    s.reply()
    s.send(f"GEN 12 temperature=0.9 top_k=20 seed=77 {csv(prompt[:20])}")
    r2 = s.reply()
    assert r1[2] == r2[2] and len(r1[2]) == 12
    s.send(f"GEN 12 temperature=0.9 top_k=20 seed=78 {csv(prompt[:20])}")
    assert s.reply()[2] != r1[2]
    # STOP is for the latest request: it ends with "cancel", short of its max_new
    s.send(f"GEN 600 {csv(prompt)}", "STOP")
    pp, resume, toks4, done = s.reply()
    assert done[4] == "cancel" and len(toks4) < 600
    # refused lines leave the process serving
    s.send("PING", "BGEN 0 5 1,2", "GEN 2000 1,2", f"GEN 2 {csv(prompt[:5])}")
    assert s.reply() == "ERR PING: not supported by fnx_serve"
    assert s.reply() == "ERR BGEN: fnx_serve runs without --batch"
    assert s.reply() == "ERR GEN: prompt + max_new exceed the context"
    assert len(s.reply()[2]) == 2
    # logit_bias reaches greedy requests too: a large bias on one token makes it every pick; taken away, the plain tokens are back
    s.send(f"GEN 4 logit_bias=77:90 {csv(prompt[:9])}", f"GEN 4 {csv(prompt[:9])}")
    assert s.reply()[2] == [77, 77, 77, 77]
    assert s.reply()[2] == plain(a, prompt[:9], 4)
    # penalties: a presence penalty that no logit can overcome forbids every token of the window, so nothing repeats
    s.send(f"GEN 24 temperature=0.8 seed=3 penalty_present=80 penalty_last_n=64 {csv(prompt[:9])}")
    got = s.reply()[2]
    assert len(got) == 24 and len(set(got)) == 24 and not set(got) & set(prompt[:9])
    assert s.quit() == 0
    a.close()
    # an end-of-sequence token from the command line ends a reply with "stop"
    s = _Serve("--native", path, "--max-context", 1024, "--spec", 3, "--lookup", 0, "--eos", want[5])
    s.line(), s.line()
    s.send(f"GEN 24 {csv(prompt)}")
    pp, resume, toks, done = s.reply()
    assert toks == want[:want.index(want[5]) + 1] and done[4] == "stop"
    assert s.quit() == 0


def test_logit_rules_change_the_window_rows(F, O, model):
    """The engine's windows under a request's logit_bias and penalties: the logits left in the window buffer are the plain
    window's logits changed by the oracle's restatement of the sampler's first stage (row j's penalty window: the kept tokens
    and window rows 0..j), and the greedy result is their argmax."""
    cfg, eng, om = model
    rng = np.random.default_rng(8)
    eng.reset()
    eng.set_logit_rules()
    prompt = rng.integers(0, 50, size=30).tolist()          # a small alphabet: tokens repeat inside the window
    eng.prefill(prompt)
    toks = rng.integers(0, 50, size=5).tolist()
    eng.verify(toks)
    plain = eng.tensor("buf.logits", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.vocab)[:5].copy()
    bias = [(3, 2.5), (int(toks[1]), -1.0), (cfg.vocab - 1, 50.0)]
    for last_n, rep, fr, pr, b in [(16, 1.3, 0.2, 0.4, bias), (64, 1.1, 0.0, 0.0, ()), (0, 1.0, 0.0, 0.0, bias), (4096, 0.8, 0.05, -0.1, bias[:1])]:
        eng.set_logit_rules(last_n, rep, fr, pr, b)
        n, path, em = eng.verify(toks)
        got = eng.tensor("buf.logits", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.vocab)[:5]
        want = O.logit_adjust(plain, prompt, toks, last_n, rep, fr, pr, b)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (last_n, rep)
        best = want.argmax(axis=1)
        k = 1
        while k < 5 and toks[k] == best[k - 1]:
            k += 1
        assert n == k and em == best[:k].tolist()
    with pytest.raises(F.FnxError, match="chains"):
        eng.set_logit_rules(8, 1.2)
        eng.verify(toks[:3], [-1, 0, 0])
    with pytest.raises(F.FnxError, match="penalty window"):
        eng.set_logit_rules(5000, 1.2)
    with pytest.raises(F.FnxError, match="bias entry"):
        eng.set_logit_rules(0, bias=[(cfg.vocab, 1.0)])
    eng.set_logit_rules()
    eng.verify(toks)
    assert np.array_equal(eng.tensor("buf.logits", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.vocab)[:5], plain)


def test_serve_process_batched_slots(F, tmp_path):
    """fnx_serve --batch: prompts read into slots, the decoding slots sharing windows (the engine's batched lanes).  Every slot's
    tokens are the plain greedy tokens of its prompt alone; BSTOP ends one slot and leaves the others; a solo GEN runs
    between windows when slot 0 is free."""
    from gguf_files import model_meta, tiny_model_tensors, write_gguf
    cfg = small_cfg(F, max_ctx=1024)
    a = F.Engine(cfg)
    a.init_synthetic(seed=9, sigma=0.02)
    path = tmp_path / "tiny.gguf"
    write_gguf(path, model_meta(cfg), tiny_model_tensors(F, a, cfg))
    rng = np.random.default_rng(33)
    prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (25, 40, 12)]

    def plain(prompt, n_new):
        a.reset()
        a.prompt(prompt[:-1])
        x, out = prompt[-1], []
        for _ in range(n_new):
            n, path_, em = a.verify([x])
            a.commit([0])
            x = em[0]
            out.append(x)
        return out

    want = [plain(p, 20) for p in prompts]
    csv = lambda ids: ",".join(map(str, ids))
    s = _Serve("--native", path, "--max-context", 1024, "--spec", 3, "--lookup", 0, "--batch", 4, "--prompt-chunk", 4096)
    assert "batch_slots=4" in s.line()
    assert s.line() == "READY 1024 stop"
    s.send(f"BGEN 1 20 {csv(prompts[0])}", f"BGEN 2 14 {csv(prompts[1])}", f"BGEN 3 1 {csv(prompts[2])}")
    got, done, adm, first = {1: [], 2: [], 3: []}, {}, {}, []
    while len(done) < 2 or len(adm) < 3:
        w = s.line().split()
        if w[0] == "T":
            first.append(int(w[1]))
        elif w[0] == "BADM":
            adm[int(w[1])] = int(w[2])
        elif w[0] == "BT":
            got[int(w[1])].append(int(w[2]))
        elif w[0] == "BDONE":
            done[int(w[1])] = w[2:]
        else:
            assert w[0] in ("PP", "RESUME", "DONE"), w
    assert adm == {1: 1, 2: 1, 3: 0}                      # max_new = 1 ends with its first token
    assert first == [want[0][0], want[1][0], want[2][0]]
    assert [first[0]] + got[1] == want[0] and [first[1]] + got[2] == want[1][:14]
    assert done[1][0] == "20" and done[1][1] == "length" and done[2][0] == "14" and int(done[1][4]) >= int(done[1][3]) >= 0
    # a slot stopped while it decodes; the other goes on to its end; a solo request in between
    s.send(f"BGEN 0 600 {csv(prompts[0])}", f"BGEN 1 30 {csv(prompts[1])}")
    seen = {0: [], 1: []}
    sent_stop = False
    done = {}
    while len(done) < 2:
        w = s.line().split()
        if w[0] == "BT":
            seen[int(w[1])].append(int(w[2]))
            if not sent_stop and len(seen[0]) >= 3:
                s.send("BSTOP 0")
                sent_stop = True
        elif w[0] == "BDONE":
            done[int(w[1])] = w[2:]
    assert done[0][1] == "cancel" and 3 <= int(done[0][0]) < 600 and done[1][1] == "length"
    assert seen[0] == want[0][1:1 + len(seen[0])] or seen[0][:19] == want[0][1:20]
    s.send(f"GEN 5 {csv(prompts[2])}")
    l = s.line()
    toks = []
    while not l.startswith("DONE"):
        if l.startswith("T "):
            toks.append(int(l.split()[1]))
        l = s.line()
    assert toks == want[2][:5]
    s.send("BGEN 7 5 1,2", "BGEN 1 5 temperature=0.5 1,2")
    assert s.line() == "ERR BGEN: no such free slot 7 (--batch 4)"
    assert s.line().startswith("ERR BGEN: batched slots decode greedily")
    assert s.quit() == 0
    a.close()


def test_serve_process_parks_and_resumes_conversations(F, tmp_path):
    """fnx_serve --conversation-cache-mib: a conversation displaced by another one waits in host memory (the engine's sequence
    state) and comes back when a later prompt goes on from it: RESUME counts its tokens and the reply is the one the
    conversation would have got had it never left the engine."""
    from gguf_files import model_meta, tiny_model_tensors, write_gguf
    cfg = small_cfg(F, max_ctx=1024)
    a = F.Engine(cfg)
    a.init_synthetic(seed=9, sigma=0.02)
    path = tmp_path / "tiny.gguf"
    write_gguf(path, model_meta(cfg), tiny_model_tensors(F, a, cfg))
    rng = np.random.default_rng(44)
    pa, pb = rng.integers(0, cfg.vocab, size=30).tolist(), rng.integers(0, cfg.vocab, size=22).tolist()
    csv = lambda ids: ",".join(map(str, ids))

    def plain_more(prompt_new, n_new):   # on engine `a`, which holds the conversation so far
        if len(prompt_new) > 1:
            a.prompt(prompt_new[:-1])
        x, out = prompt_new[-1], []
        for _ in range(n_new):
            n, path_, em = a.verify([x])
            a.commit([0])
            x = em[0]
            out.append(x)
        return out

    s = _Serve("--native", path, "--max-context", 1024, "--spec", 3, "--lookup", 4, "--prompt-chunk", 4096, "--conversation-cache-mib", 64)
    assert "conversation_cache_mib=64" in s.line()
    s.line()
    s.send(f"GEN 8 {csv(pa)}")
    _, resume, ta, _ = s.reply()
    a.reset()
    assert resume == 0 and ta == plain_more(pa, 8)
    s.send(f"GEN 6 {csv(pb)}")                       # another conversation: A is parked
    _, resume, tb, _ = s.reply()
    assert resume == 0 and len(tb) == 6
    more = pa + ta + rng.integers(0, cfg.vocab, size=5).tolist()
    s.send(f"GEN 7 {csv(more)}")                     # A goes on: its state comes back from host memory (B is parked in turn)
    _, resume, ta2, done = s.reply()
    assert resume == len(pa) + len(ta) - 1 and done[7] == str(resume)
    assert ta2 == plain_more(more[len(pa) + len(ta) - 1:], 7)
    moreb = pb + tb + [int(rng.integers(0, cfg.vocab))]
    s.send(f"GEN 3 {csv(moreb)}")                    # and B likewise
    _, resume, tb2, _ = s.reply()
    assert resume == len(pb) + len(tb) - 1 and len(tb2) == 3
    assert s.quit() == 0
    a.close()
