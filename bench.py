"""Benchmark of the speculative-decoding verify path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1): the full synthetic 48-layer model (hidden 2048, 512 experts top-10 + shared expert, every 4th layer
gated attention, the rest gated DeltaNet, vocab 151,936, one MTP layer), random-init weights quantised to IQ3_S,
a 4,096-token uniform-random context, k + 1 = 5 rows per window.  A step is one decode round: the MTP draft chain
(4 calls), one verify window, greedy acceptance, commit.  Drafts: the sequence's own greedy continuation (computed
before the timed region), each draft wrong with probability 0.28 (seeded), which gives the acceptance the reference
reports for its MTP drafts (docs/SWITCHES.md:81) - the reference's `spec` test mode (engine/tools/fnx_run.cpp:8-9);
the MTP chain is still computed and timed every round.

value    decode tok/s from the device times of the round's graphs (inputs resident on the GPU)
e2e      the same through Engine.verify / commit / draft with host token buffers: H2D of the window's tokens and
         D2H of the acceptance result inside the timed region
roofline the routed-expert gate|up kernel (the dominant kernel) timed live with CUDA events over all 48 layers'
         weights; plus the whole verify step against its compulsory bytes
N > 1:   expert-parallel ranks (512 experts split evenly, one exchange per layer over NVLink peer memory, or NCCL with
         FNX_EP_NCCL=1), same token stream on every rank, device-timed, max over ranks ("strong" scaling: the work is fixed).
Other configurations: --config 2 (tree windows with lookup drafts), 3 (cold prefill of 38,912 tokens on the prompt pass),
4 (8 sequences x 131,072-token contexts in batched lanes; also a sub-object of the default run).  Side modes, not bench
lines: --prefill-moe T, --attn-prompt T, --verify-only.
"""
from __future__ import annotations

import argparse
import datetime
import json
import signal
import zlib
import os
import pathlib
import statistics
import subprocess
import sys
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

METRIC = "decode tok/s (MTP+lookup spec verify), verify-step us, % of HBM roofline"
CTX, K_DRAFT, P_BAD = 4096, 4, 0.28
C2_CTX, C2_LOOKUP = 32768, 15            # configuration 2: context and the longest lookup branch
C3_TOKENS = 38912                          # configuration 3: the cold prompt
C4_CTX, C4_SEQS, C4_LANES = 131072, 8, 4   # configuration 4: context per sequence, sequences, lanes per window
E_B = 1351680          # bytes of one expert: (2*512*2048 + 2048*512) * 110 / 256
# DRAM bytes per expert job of the gate|up launch, from an ncu capture of one launch (dram__bytes_read.sum +
# dram__bytes_write.sum = 42.02 MB for 46 jobs; the algorithmic figure is 901,120 bytes per job)
NCU_TRAFFIC_PER_JOB = 42.02e6 / 46


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class Clocks:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.idx, self.t0 = [], None, gpu_index, None

    def launch(self):
        """Starts the sampler (it needs a few hundred ms before its first line); mark() opens the timed region."""
        q = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "20", "-i", str(self.idx)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def start(self):
        if self.proc is None:
            self.launch()
        self.t0 = time.time()

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        t1 = time.time()
        time.sleep(0.05)
        self.proc.terminate()
        out = self.proc.communicate()[0]
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                if self.t0 is not None and not (self.t0 - 0.02 <= ts <= t1 + 0.02):
                    continue   # outside the timed region
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# the draft layer's head covers a draft vocabulary, as the reference's does (its English one holds 40,525 ids; rounded up to
# whole 16-row tiles); the ids are synthetic: spread evenly over the vocabulary
DRAFT_VOCAB = 40528


def model_config(F, ep_rank, ep_size, layers=48, rounds=64, ctx=CTX):
    # room for the context, every round's window of k + 1 rows, and the few single-row windows run afterwards
    room = max(1024, (rounds + 8) * (K_DRAFT + 1) + 64)
    return F.flash_next_config(n_layer=layers, max_ctx=ctx + (room + 255) // 256 * 256, max_rows=32, ep_rank=ep_rank, ep_size=ep_size, draft_vocab=DRAFT_VOCAB)


def step_bytes(routed_jobs_per_step: float, ctx: int, T: int):
    """Algorithmic bytes of one verify step: primary = active experts + attention K/V (the target's definition);
    all = every compulsory byte (router, dense projections, DeltaNet state, head)."""
    kv = 12 * ((ctx + T) * 2 * 256 * 2 * 2 + T * 2 * 256 * 2 * 2)
    primary = (routed_jobs_per_step + 48) * E_B + kv
    blk = 110 / 256
    dense = 12 * (9216 * 2048 + 2048 * 4096) * blk + 36 * (12352 * 2048 + 2048 * 4096) * blk
    router = 48 * 513 * 2048 * 4
    state = 36 * (1 + T) * 32 * 128 * 128 * 4
    head = 151936 * 2048 * blk
    return primary, primary + dense + router + state + head


def cpu_leg(F, O, steps, threads):
    """The CPU restatement on the host cores, on a bounded sample, and the full-size parity check that comes with it.

    A four-layer engine of the benchmark model's own dimensions (three DeltaNet layers and one attention layer, random
    init, seed 0) is mirrored by the oracle.  Parity: one 5-row window after a short prompt, engine against oracle
    (routing indices, hidden states, logits, accepted tokens).  Timing: the oracle's DeltaNet layer and attention layer
    (each with router, routed and shared experts) and the head on a 5-row window at the benchmark's context (the
    attention cache filled with random f16 rows); a full 48-layer step is 36 x the first + 12 x the second + the head.
    Returns (per-sample dicts, parity dict)."""
    import numpy as np
    import torch
    from helpers import OracleModel, rel_err
    used = O.threads(threads)
    cfg = F.flash_next_config(n_layer=4, max_ctx=CTX + 256, max_rows=8)
    eng = F.Engine(cfg)
    eng.init_synthetic(seed=0, sigma=0.02)
    om = OracleModel(F, O, eng, cfg, with_mtp=False)
    rng = np.random.default_rng(1)
    # ---- parity at the benchmark's dimensions
    prompt = rng.integers(0, cfg.vocab, size=12).tolist()
    eng.reset()
    eng.prefill(prompt)
    for i in range(0, len(prompt), cfg.max_rows):
        w = prompt[i:i + cfg.max_rows]
        om.verify(w, None)
        om.commit(list(range(len(w))))
    T = 1 + K_DRAFT
    for _ in range(8):   # the first seeded window without a routing near-tie (top-K is discontinuous)
        toks = rng.integers(0, cfg.vocab, size=T).tolist()
        want = om.verify(toks, None)
        gaps = [np.sort(lg[t, :-1])[::-1][cfg.top_k - 1:cfg.top_k + 1] for _, lg in om.routing for t in range(T)]
        if min(float(g[0] - g[1]) for g in gaps) > 2e-4 * max(1.0, max(float(np.abs(lg).max()) for _, lg in om.routing)):
            break
    got = eng.verify(toks)
    R = eng.tensor("buf.R", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.hidden)[:T]
    logits = eng.tensor("buf.logits", torch.float32).cpu().numpy().reshape(cfg.max_rows, cfg.vocab)[:T]
    topi = eng.tensor("buf.topi", torch.int32).cpu().numpy().reshape(cfg.max_rows, cfg.top_k)[:T]
    parity = {"what": "4 layers of the benchmark model's dimensions (512 experts, hidden 2048, vocab 151936), 5-row window after a 12-token prompt, engine vs CPU oracle",
              "rel_err_hidden": rel_err(R, om.R), "rel_err_logits": rel_err(logits, om.logits),
              "routing_exact": bool(np.array_equal(topi, om.routing[-1][0])),
              "accepted_exact": got == (want[0], list(want[1]), list(want[2]))}
    assert parity["routing_exact"] and parity["accepted_exact"] and parity["rel_err_hidden"] < 2e-3 and parity["rel_err_logits"] < 2e-3, parity
    eng.close()
    # ---- timing sample
    L = om.layers[3]
    L["kc"][:CTX] = rng.standard_normal((CTX, om.nkv, om.hd)).astype(np.float16).view(np.uint16)
    L["vc"][:CTX] = rng.standard_normal((CTX, om.nkv, om.hd)).astype(np.float16).view(np.uint16)
    om.pos = CTX
    R0 = rng.standard_normal((1 + K_DRAFT, om.H)).astype(np.float32)
    out = []
    for _ in range(steps):
        t0 = time.perf_counter()
        R = om._gdn(om.layers[0], R0, None)
        R = om._moe(om.layers[0], R)
        t1 = time.perf_counter()
        R = om._attention(om.layers[3], R, om.pos, None, None)
        R = om._moe(om.layers[3], R)
        t2 = time.perf_counter()
        lg = O.iq3s_gemv(om.head, om.V, om.H, O.rmsnorm(R, om.out_norm, cfg.eps))
        O.argmax(lg)
        t3 = time.perf_counter()
        out.append({"sampled_s": t3 - t0, "step_s": 36 * (t1 - t0) + 12 * (t2 - t1) + (t3 - t2)})
    return out, parity, used


CPU_SAMPLE = ("per step: 1 DeltaNet layer + 1 attention layer (each with router, routed + shared experts) + the head of the benchmark model on the host "
              "cores, 5-row window at ctx 4096; a verify step = 36 x the first + 12 x the second + the head (extrapolated); MTP chain not included")


def ep_setup(F, eng, rank, world):
    """Expert-parallel ranks: the NCCL communicator and, unless FNX_EP_NCCL=1, the per-layer sum over NVLink peer memory
    (fused with the combine): the ranks exchange their IPC handles.  Returns whether the peer-memory sum is in use."""
    if world == 1:
        return False
    import ctypes as C
    import torch
    import torch.distributed as dist
    uid = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        buf = (C.c_char * 128)()
        F.check(F.lib().fnx_comm_unique_id(buf))
        uid = torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8).clone()
    uid = uid.cuda()
    dist.broadcast(uid, 0)
    raw = bytes(uid.cpu().numpy().tobytes())
    F.check(F.lib().fnx_engine_comm_init(eng._h, raw, rank, world))
    use_peer = os.environ.get("FNX_EP_NCCL", "0") != "1"
    if use_peer:
        mine = (C.c_char * 128)()
        F.check(F.lib().fnx_engine_ep_handles(eng._h, mine))
        hm = torch.frombuffer(bytearray(mine.raw), dtype=torch.uint8).clone().cuda()
        allh = [torch.zeros(128, dtype=torch.uint8, device="cuda") for _ in range(world)]
        dist.all_gather(allh, hm)
        blob = b"".join(bytes(t.cpu().numpy().tobytes()) for t in allh)
        F.check(F.lib().fnx_engine_ep_open(eng._h, blob, rank, world))
    return use_peer


def _max_over_ranks(world, vals):
    import torch
    if world == 1:
        return vals
    t = torch.tensor(vals, device="cuda", dtype=torch.float64)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return [float(v) for v in t]


def _barrier(world):
    import torch
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def run_config4(a, F, eng, cfg, rank, world, local, use_peer, emit=True):
    """Configuration 4: 8 concurrent sequences, each at a 131,072-token context, MTP drafts of k = 4, the sampling rule at
    temperature 0.7 with seeded Philox uniforms; expert-parallel over the ranks.  The sequences run as batched lanes: two
    windows of four lanes (5 rows each) per round.  A step = one round of all 8 sequences: per window the MTP draft chain
    over its lanes, the verify window, acceptance, commit.  The contexts are synthetic: seeded random K/V rows and DeltaNet
    states stand in for 8 x 131,072 prefilled tokens (the values do not change the step's cost)."""
    import numpy as np
    import torch
    ctx = a.ctx if a.ctx != CTX else C4_CTX
    g = torch.Generator(device="cuda")
    g.manual_seed(4)
    for l in range(a.layers):
        attn = (l + 1) % cfg.attn_every == 0
        if attn:
            for nm in ("k_cache", "v_cache"):
                t = eng.tensor(f"l{l}.{nm}", torch.float16)
                for o in range(0, t.numel(), 1 << 28):   # in pieces of 2^28 elements
                    t[o:o + (1 << 28)].normal_(0.0, 1.0, generator=g)
        else:
            eng.tensor(f"l{l}.state", torch.float32).normal_(0.0, 0.02, generator=g)
            eng.tensor(f"l{l}.conv_hist", torch.float32).normal_(0.0, 0.5, generator=g)
    for nm in ("k_cache", "v_cache"):
        eng.tensor(f"mtp.{nm}", torch.float16).normal_(0.0, 1.0, generator=g)
    for s in range(C4_SEQS):
        eng.set_position(s, ctx)
    samp = F.Sampling(0.7, 1.0, 0.0, 0)
    eng.set_sampling(samp, seed=4)
    rng = np.random.default_rng(4)
    groups = [list(range(i, min(i + C4_LANES, C4_SEQS))) for i in range(0, C4_SEQS, C4_LANES)]
    nxt = {s: int(rng.integers(0, cfg.vocab)) for s in range(C4_SEQS)}
    pending = [None] * len(groups)
    clocks = Clocks(local)
    clocks.launch()
    est = torch.cuda.ExternalStream(F.lib().fnx_engine_stream(eng._h))
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dev_ms = verify_ms = 0.0
    tokens = accepted = offered = 0
    stream = []
    c0 = None
    for r in range(a.warmup + a.steps):
        if r == a.warmup:
            _barrier(world)
            c0 = eng.counters()
            clocks.start()
            t0.record(est)
            wall0 = time.perf_counter()
        for gi, grp in enumerate(groups):
            # (the window buffers are shared by the groups: a group's drafts for its NEXT window are taken right after its commit)
            drafts = pending[gi] if pending[gi] is not None else [rng.integers(0, cfg.vocab, size=K_DRAFT).tolist() for _ in grp]
            res = eng.verify_lanes(grp, [[nxt[s]] + drafts[j] for j, s in enumerate(grp)])
            if r >= a.warmup:
                dev_ms += eng.last_ms()
                verify_ms += eng.last_ms()
            eng.commit_lanes(grp, [x[0] for x in res])
            pending[gi] = eng.draft_lanes(grp, K_DRAFT)
            if r >= a.warmup:
                dev_ms += eng.last_ms()
            for j, s in enumerate(grp):
                n, _, em = res[j]
                nxt[s] = em[-1]
                stream.extend(em)
                if r >= a.warmup:
                    tokens += n
                    accepted += n - 1
                    offered += K_DRAFT
    t1.record(est)
    _barrier(world)
    wall = time.perf_counter() - wall0
    clk = clocks.stop()
    c1 = eng.counters()
    dev_ms, e2e_ms = _max_over_ranks(world, [dev_ms, t0.elapsed_time(t1)])
    T = C4_LANES * (1 + K_DRAFT)
    jobs_per_window = (c1[1] - c0[1]) / max(1, c1[2] - c0[2]) * a.layers if c1[2] > c0[2] else 0.0
    kv = 12 * C4_LANES * ((ctx + 5) * 2 * 256 * 2 * 2)
    line = {"metric": METRIC, "value": tokens / (dev_ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": dev_ms / a.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8xint3->f32", "data": "synthetic",
            "config": {"workload": (f"configuration 4: {C4_SEQS} concurrent sequences at ctx {ctx} each (synthetic: seeded random K/V rows and DeltaNet states, seed 4), MTP k={K_DRAFT} "
                                    f"drafts from the draft layer, sampling rule at temperature 0.7 (Philox, seed 4), batched lanes: {len(groups)} windows of {C4_LANES} lanes x "
                                    f"{1 + K_DRAFT} rows per round; experts sharded over the ranks"),
                       "timing": "per-step K/V reads (tens of GB) and expert weights far larger than the 126 MB L2; CUDA events on the engine's stream",
                       "parallelism": f"ep{world}", "layers": a.layers},
            "clocks": clk, "gpu_launches": int(c1[0] - c0[0]),
            "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": len(groups) * (4 * T + 4 * (2 * C4_LANES + 1) + 4 * C4_LANES * 2),
                    "d2h_bytes_per_step": len(groups) * (4 * C4_LANES * 65 + 4 + 4 * C4_LANES * K_DRAFT), "wall_ms_per_step": wall * 1e3 / a.steps},
            "verify_window_us": verify_ms * 1e3 / (a.steps * len(groups)), "accepted_per_offered": accepted / max(1, offered), "tokens_per_step": tokens / a.steps,
            "tokens_crc": zlib.crc32(np.asarray(stream, np.int64).tobytes()), "ep_sum": "none" if world == 1 else ("peer-memory" if use_peer else "nccl"),
            "window_bytes": {"kv_read": kv, "routed_jobs_per_window": jobs_per_window, "expert_bytes": (jobs_per_window + a.layers * 5) * E_B / max(1, world)}}
    eng.close()
    if not emit:
        return line
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0


def run_config3(a, F, eng, cfg, rank, world, local, use_peer):
    """Configuration 3: cold prefill of 38,912 uniform-random tokens (seed 3).  One rank reads the prompt on the prompt pass
    (fnx_engine_prompt: projections, experts and attention on the tensor cores, the DeltaNet scan); expert-parallel
    ranks, and `--prompt-windows`, read it through chained 32-row windows of the decode kernels.  One step = the whole prompt."""
    import numpy as np
    import torch
    n = a.ctx if a.ctx != CTX else C3_TOKENS
    toks = np.random.default_rng(3).integers(0, cfg.vocab, size=n).tolist()
    est = torch.cuda.ExternalStream(F.lib().fnx_engine_stream(eng._h))
    windows = world > 1 or a.prompt_windows
    clocks = Clocks(local)
    clocks.launch()
    times, walls = [], []
    c0 = eng.counters()
    for it in range(1 + max(1, min(a.steps, 2))):   # one warm-up pass (graph capture), then the timed passes
        eng.reset()
        _barrier(world)
        if it == 1:
            clocks.start()
            c0 = eng.counters()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.perf_counter()
        t0.record(est)
        if windows:
            eng.prefill(toks)
        else:
            eng.prompt(toks)
        t1.record(est)
        _barrier(world)
        walls.append(time.perf_counter() - w0)
        times.append(t0.elapsed_time(t1))
    clk = clocks.stop()
    c1 = eng.counters()
    ms = _max_over_ranks(world, [min(times[1:])])[0]
    wall = min(walls[1:])
    passes = len(times) - 1
    phases, roof = None, None
    if not windows:
        # one more pass, untimed as a whole, with the phases timed by events: the tensor-core products against the dense peak
        eng.prompt_timing(True)
        eng.reset()
        eng.prompt(toks)
        phases = eng.prompt_timing(False)
        pk = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
        peak = float(pk.get("bf16_tflops_sustained", pk.get("bf16_tflops", 1400.0)))
        L, H, Fn = a.layers, cfg.hidden, cfg.ffn
        n_attn = sum(1 for l in range(L) if (l + 1) % cfg.attn_every == 0)
        q_rows, kv_rows = cfg.n_q_head * 2 * cfg.head_dim, cfg.n_kv_head * cfg.head_dim
        gdn_in = (2 * cfg.gdn_k_head + cfg.gdn_v_head) * cfg.gdn_head_dim + cfg.gdn_v_head * cfg.gdn_head_dim + 2 * cfg.gdn_v_head
        fl = {"experts": 2.0 * n * (cfg.top_k + 1) * 3 * H * Fn * L,
              "in_proj": 2.0 * n * H * (n_attn * (q_rows + 2 * kv_rows) + (L - n_attn) * gdn_in),
              "out_proj": 2.0 * n * H * (n_attn * cfg.n_q_head * cfg.head_dim + (L - n_attn) * cfg.gdn_v_head * cfg.gdn_head_dim),
              "attention": 4.0 * cfg.n_q_head * cfg.head_dim * (n * (n + 1) / 2.0) * n_attn}
        tf = {k: fl[k] / (phases[k] * 1e-3) / 1e12 for k in fl if phases.get(k, 0) > 0}
        roof = {"bound": "tensor", "kernel": "k_gemm_tma_jobs (grouped expert products on tcgen05.mma, operands by tensor copies; the phase also decodes the experts to f16, copies the rows into job order and combines)", "achieved": tf.get("experts"), "peak": peak, "unit": "TFLOP/s",
                "frac": tf.get("experts", 0.0) / peak, "peak_kind": "measured (sustained)" if pk else "fallback", "traffic": None,
                "tflops_by_phase": tf, "note": "device ms per phase from CUDA events around the phases of every layer and chunk, in an extra pass of the same prompt; "
                "projections, experts and attention run on tcgen05.mma"}
    line = {"metric": "prefill tok/s (cold prompt)", "value": n / (ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": passes, "warmup": 1, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8xint3->f32", "data": "synthetic",
            "config": {"workload": f"configuration 3: cold prefill of {n} uniform-random tokens (seed 3) " +
                       ("through chained 32-row windows of the decode kernels" if windows else "on the prompt pass (projections, experts and attention on tcgen05.mma, DeltaNet as conv / scan / norm)"),
                       "timing": "weights (17 GB) and activations far larger than the 126 MB L2; CUDA events on the engine's stream", "parallelism": f"ep{world}", "layers": a.layers},
            "clocks": clk, "gpu_launches": int((c1[0] - c0[0]) / passes),
            "e2e": {"value": n / wall, "unit": "tok/s", "h2d_bytes_per_step": 4 * n + 4 * n, "d2h_bytes_per_step": 0, "wall_ms_per_step": wall * 1e3},
            "windows": (n + cfg.max_rows - 1) // cfg.max_rows, "us_per_window": ms * 1e3 / ((n + cfg.max_rows - 1) // cfg.max_rows),
            "path": "windows" if windows else "prompt pass", "phases_ms": phases, "roofline": roof}
    if rank == 0:
        print(json.dumps(line))
    eng.close()
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0


def edit_like_context(n, vocab, seed):
    """Configuration 2's context: uniform-random tokens in which 60% of the positions are copies of earlier spans of
    length 20-200 (an edit-like workload)."""
    import numpy as np
    rng = np.random.default_rng(seed)
    out = rng.integers(0, vocab, size=n).tolist()
    i = 256
    while i < n:
        if rng.random() < 0.6:
            ln = int(rng.integers(20, 201))
            src = int(rng.integers(0, max(1, i - ln)))
            ln = min(ln, n - i)
            out[i:i + ln] = out[src:src + ln]
            i += ln
        else:
            i += int(rng.integers(20, 201) * 0.4 / 0.6) + 1
    return out


def run_config2(a, F, eng, cfg, rank, world, local, use_peer):
    """Configuration 2: tree verification of an MTP chain of 4 plus a prompt-lookup branch of up to 15 tokens (3-gram match on
    the GPU over the sequence's own 32,768-token edit-like context), greedy acceptance, rollback to the last accepted node.
    A step = the MTP draft chain, the lookup, one tree window (root + chain + branch), acceptance, commit.  The text being
    generated continues the edit-like context: the chain's drafts are the real draft layer's, the branch is what the
    drafter finds."""
    import numpy as np
    import torch
    ctx = a.ctx if a.ctx != CTX else C2_CTX
    total = a.warmup + a.steps
    full = edit_like_context(ctx + total + 1, cfg.vocab, 2)
    eng.reset()
    eng.prefill(full[:ctx])
    clocks = Clocks(local)
    clocks.launch()
    est = torch.cuda.ExternalStream(F.lib().fnx_engine_stream(eng._h))
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dev_ms = verify_ms = 0.0
    tokens = rows = lk_rows = lk_kept = 0
    stream = []
    have_kept = False
    for r in range(total):
        if r == a.warmup:
            _barrier(world)
            c0 = eng.counters()
            clocks.start()
            t0.record(est)
            wall0 = time.perf_counter()
        # The text being written is the edit-like text itself: each window's root is its next token (a random-init model
        # would not continue copied spans, and then the drafter would never find a match).  The window keeps what greedy
        # acceptance keeps of the drafts; the following root is again the text's.
        x = full[ctx + r]
        chain = []
        if have_kept:
            chain = eng.draft(K_DRAFT)
            if r >= a.warmup:
                dev_ms += eng.last_ms()
        lk = eng.lookup(C2_LOOKUP, root=x)
        toks = [x] + chain + lk
        par = [-1] + list(range(0, len(chain))) + ([0] + list(range(1 + len(chain), len(chain) + len(lk))) if lk else [])
        n, path, em = eng.verify(toks, par)
        if r >= a.warmup:
            dev_ms += eng.last_ms()
            verify_ms += eng.last_ms()
            tokens += n
            rows += len(toks)
            lk_rows += len(lk)
            lk_kept += sum(1 for p in path if p > len(chain))
        # keep the root only and go on with the text's next token: the context stays the edit-like text
        eng.commit([0])
        have_kept = True
        stream.extend(em)
        x = full[ctx + r + 1]
    t1.record(est)
    _barrier(world)
    wall = time.perf_counter() - wall0
    clk = clocks.stop()
    c1 = eng.counters()
    dev_ms, e2e_ms = _max_over_ranks(world, [dev_ms, t0.elapsed_time(t1)])
    line = {"metric": METRIC, "value": tokens / (dev_ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": dev_ms / a.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8xint3->f32", "data": "synthetic",
            "config": {"workload": (f"configuration 2: tree windows (root + MTP chain of {K_DRAFT} + prompt-lookup branch of up to {C2_LOOKUP}) over a {ctx}-token edit-like context "
                                    "(seed 2: 60% of positions copy earlier spans of 20-200 tokens), greedy acceptance, rollback to the last accepted node"),
                       "timing": "inputs far larger than the 126 MB L2; CUDA events on the engine's stream", "parallelism": f"ep{world}", "layers": a.layers},
            "clocks": clk, "gpu_launches": int(c1[0] - c0[0]),
            "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": 4 * 2 * 20 + 16, "d2h_bytes_per_step": 4 * 65 + 4 + 4 * K_DRAFT + 4 * 34,
                    "wall_ms_per_step": wall * 1e3 / a.steps},
            "verify_window_us": verify_ms * 1e3 / a.steps, "rows_per_window": rows / a.steps, "lookup_rows_per_window": lk_rows / a.steps,
            "lookup_rows_kept_per_window": lk_kept / a.steps, "tokens_per_step": tokens / a.steps,
            "tokens_crc": zlib.crc32(np.asarray(stream, np.int64).tobytes()), "ep_sum": "none" if world == 1 else ("peer-memory" if use_peer else "nccl"),
            "note": ("each window's root is the next token of the edit-like text and only the root is kept (a random-init model does not continue copied spans): "
                     "tokens_per_step counts what greedy acceptance accepted, the windows' cost is that of full tree windows with real lookup branches")}
    if rank == 0:
        print(json.dumps(line))
    eng.close()
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0


def bench_config(workload, world, layers):
    """The `config` object of both arms' JSON lines (same keys, so that the two lines name the same workload)."""
    return {"workload": workload, "timing": "inputs (34 GB of weights per step cycle) far larger than the 126 MB L2; CUDA events on the engine's stream",
            "parallelism": f"ep{world}", "layers": layers, "draft_vocab": DRAFT_VOCAB}


def main():
    # a multi-rank run that stalls (a rank that never arrives) ends by itself instead of holding the GPUs
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 and hasattr(signal, "alarm"):
        signal.alarm(int(os.environ.get("FNX_BENCH_LIMIT_S", "540")))
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed steps (default 50; configuration 2: 300, so that the timed text runs through several copied spans and gaps)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", type=int, default=1, choices=[1, 2, 3, 4],
                    help="the benchmark configuration: 1 = 5-row chain windows at ctx 4096 (the headline), 3 = cold prefill of 38,912 tokens, 2 = tree windows of an MTP chain + a prompt-lookup "
                         "branch over a 32,768-token edit-like context, 4 = 8 concurrent sequences at ctx 131,072 with the sampling rule (batched lanes)")
    ap.add_argument("--layers", type=int, default=48, help="fewer layers for a quick functional run (not a valid bench number)")
    ap.add_argument("--ctx", type=int, default=CTX, help="context length (the benchmark's is 4096)")
    ap.add_argument("--prefill-moe", type=int, default=0, metavar="T",
                    help="side measurement: the prompt-sized MoE block (tcgen05 grouped expert GEMM) of layer 0 over T random rows")
    ap.add_argument("--attn-prompt", type=int, default=0, metavar="T", help="side mode: the prompt attention alone, T rows at position --ctx")
    ap.add_argument("--prompt-windows", action="store_true", help="configuration 3: read the prompt through 32-row windows of the decode kernels instead of the prompt pass")
    ap.add_argument("--no-config4", action="store_true", help="skip the 8-sequence side measurement that follows the headline run")
    ap.add_argument("--verify-only", action="store_true", help="profiling aid: prefill, then warmup + steps verify windows of k+1 rows and nothing else")
    a = ap.parse_args()
    if a.steps is None:
        a.steps = 300 if a.config == 2 else 50
    a.warmup = max(a.warmup, 3) if a.impl == "b200" else a.warmup

    import numpy as np
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if a.impl == "reference" and rank != 0:
        return 0
    import fnx_b200 as F
    torch.cuda.set_device(local)
    if world > 1 and a.impl == "b200":
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    hbm_peak, peak_kind = peaks()
    workload = (f"verify step of the synthetic 48-layer Qwen3-Next-style model (IQ3_S, seed 0), ctx {CTX} uniform-random tokens (seed 1), "
                f"k+1={1 + K_DRAFT} rows (1 committed + {K_DRAFT} drafts), greedy; drafts = own greedy continuation, each wrong with p={P_BAD}")
    if a.impl != "reference":
        if a.config == 4:
            ctx4 = a.ctx if a.ctx != CTX else C4_CTX
            room = (a.warmup + a.steps + 8) * (K_DRAFT + 1) + 64
            cfg = F.flash_next_config(n_layer=a.layers, max_ctx=ctx4 + (room + 255) // 256 * 256, max_rows=C4_LANES * (1 + K_DRAFT), ep_rank=rank, ep_size=world,
                                      n_seq=C4_SEQS, draft_vocab=DRAFT_VOCAB)
        elif a.config == 2:
            ctx2 = a.ctx if a.ctx != CTX else C2_CTX
            cfg = model_config(F, rank, world, a.layers, a.warmup + a.steps, ctx2)
        elif a.config == 3:
            cfg = model_config(F, rank, world, a.layers, 8, a.ctx if a.ctx != CTX else C3_TOKENS)
        else:
            cfg = model_config(F, rank, world, a.layers, a.warmup + a.steps, a.ctx)
        eng = F.Engine(cfg)
        eng.init_synthetic(seed=0, sigma=0.02)
    use_peer = ep_setup(F, eng, rank, world) if a.impl == "b200" else False
    if a.config == 4:
        return run_config4(a, F, eng, cfg, rank, world, local, use_peer)
    if a.config == 2:
        return run_config2(a, F, eng, cfg, rank, world, local, use_peer)
    if a.config == 3:
        return run_config3(a, F, eng, cfg, rank, world, local, use_peer)
    if a.attn_prompt:
        # config 3's attention on its own: T prompt rows at position --ctx against a random f16 cache (a profiling aid)
        T, pos0 = a.attn_prompt, a.ctx
        nq, nkv, hd = cfg.n_q_head, cfg.n_kv_head, cfg.head_dim
        kc = torch.randn((pos0 + T + 8, nkv, hd), device="cuda").half().view(torch.int16)
        vc = torch.randn((pos0 + T + 8, nkv, hd), device="cuda").half().view(torch.int16)
        qg = torch.randn((T, nq, 2 * hd), device="cuda")
        pos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
        res = {}
        for form, mma_sync, rows_per_block in (("tcgen05", False, 16), ("mma_sync", True, 12)):
            for _ in range(max(a.warmup, 1)):
                F.attn_prompt(qg, kc, vc, pos, mma_sync=mma_sync)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.steps):
                F.attn_prompt(qg, kc, vc, pos, mma_sync=mma_sync)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / a.steps
            flop = 4.0 * hd * nq * (pos0 * T + T * (T + 1) / 2)
            res[form] = {"ms": ms, "tflops": flop / ms / 1e9, "kv_gbs": (pos0 + T / 2) * nkv * hd * 4 * ((T + rows_per_block - 1) // rows_per_block) / ms / 1e6}
        print(json.dumps({"mode": "attn-prompt", "rows": T, "position": pos0, **res,
                          "note": "fnx_attn_prompt, both forms; kv_gbs = cache bytes the blocks read (from L2 mostly) per second"}))
        return
    if a.prefill_moe:
        # config 3's expert path on one layer: T rows grouped by expert, gate|up + SwiGLU + down on the tensor cores
        T = a.prefill_moe
        x = torch.randn((T, cfg.hidden), device="cuda")
        nw = torch.ones(cfg.hidden, device="cuda")
        wr = eng.tensor("l0.router", torch.float32).view(cfg.n_expert + 1, cfg.hidden)
        topi, topw, logits = F.route_rows(wr, x, cfg.top_k, norm_w=nw)
        wgu, wdn = eng.tensor("l0.experts_gu", torch.uint8), eng.tensor("l0.experts_dn", torch.uint8)
        sgu, sdn = eng.tensor("l0.shared_gu", torch.uint8), eng.tensor("l0.shared_dn", torch.uint8)
        scratch = torch.empty(F.lib().fnx_moe_prefill_scratch_bytes(T, cfg.top_k, cfg.n_expert, cfg.hidden, cfg.ffn), dtype=torch.uint8, device="cuda")
        out = torch.zeros((T, cfg.hidden), device="cuda")
        err = F.new_err()
        run = lambda: F.moe_prefill(wgu, wdn, sgu, sdn, topi, topw, logits, x, cfg.ffn, norm_w=nw, out=out, scratch=scratch, err=err)
        for _ in range(max(a.warmup, 1)):
            run()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            run()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / a.steps
        pairs = T * (cfg.top_k + 1)
        flops = pairs * 6.0 * cfg.hidden * cfg.ffn
        pk = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
        tf_peak = float(pk.get("bf16_tflops", 1590.0))
        print(json.dumps({"mode": "prefill-moe", "rows": T, "ms_per_block": ms, "rows_per_s": T / ms * 1e3, "tflops": flops / ms / 1e9,
                          "peak_tflops": tf_peak, "peak_kind": "measured" if pk else "fallback", "frac": flops / ms / 1e9 / tf_peak,
                          "err": int(err.item()), "note": "one layer's routed + shared experts; routing given; includes the job build (the job count stays on the device)"}))
        return
    if a.impl == "reference":
        import oracle as O
        cores = os.cpu_count() or 1
        samples, parity, used = cpu_leg(F, O, a.warmup + a.steps, cores)
        samples = samples[a.warmup:]
        t_step = sum(s["step_s"] for s in samples) / len(samples)
        t_sampled = sum(s["sampled_s"] for s in samples) / len(samples)
        # expected tokens per round at the drafts' acceptance: 1 + p + p^2 + ...
        exp_tok = sum((1 - P_BAD) ** j for j in range(K_DRAFT + 1))
        v = exp_tok / t_step
        line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "tok/s", "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup,
                "ms_per_step": t_sampled * 1e3, "extrapolated": True, "extrapolated_step_ms": t_step * 1e3,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8xint3->f32",
                "data": "synthetic", "config": bench_config(workload, a.gpus, a.layers),
                "cpu_baseline": {"value": v, "unit": "tok/s", "cores": used, "host_cores": cores, "kind": "port", "sample": CPU_SAMPLE,
                                 "extrapolated": True, "scaling": "36 x DeltaNet layer + 12 x attention layer + 1 x head", "sampled_ms_per_step": t_sampled * 1e3},
                "parity_full_size": parity,
                "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return 0

    rng = np.random.default_rng(1)
    prompt = rng.integers(0, cfg.vocab, size=a.ctx + 1).tolist()
    total_rounds = a.warmup + a.steps
    if a.verify_only:
        eng.reset()
        eng.prefill(prompt[:-1])
        row = [prompt[-1]] + rng.integers(0, cfg.vocab, size=K_DRAFT).tolist()
        ts = []
        for _ in range(total_rounds):
            eng.verify(row)
            ts.append(eng.last_ms())
        print(json.dumps({"mode": "verify-only", "layers": a.layers, "ctx": a.ctx, "verify_step_us": statistics.median(ts[a.warmup:]) * 1e3}))
        eng.close()
        return 0

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    # ---- the greedy continuation the drafts are taken from (not timed)
    eng.reset()
    eng.prefill(prompt[:-1])
    x, want = prompt[-1], []
    for _ in range(total_rounds * (K_DRAFT + 1) + K_DRAFT):
        n, path, em = eng.verify([x])
        eng.commit([0])
        x = em[0]
        want.append(x)
    # ---- the decode rounds
    eng.reset()
    eng.prefill(prompt[:-1])
    bad = np.random.default_rng(2).random((total_rounds, K_DRAFT)) < P_BAD
    x, done = prompt[-1], 0
    dev_ms, tokens, accepted, offered = 0.0, 0, 0, 0
    c0 = None
    clocks = Clocks(local)
    clocks.launch()
    t_ev0, t_ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    est = torch.cuda.ExternalStream(F.lib().fnx_engine_stream(eng._h))
    have_kept = False
    for r in range(total_rounds):
        if r == a.warmup:
            barrier()
            c0 = eng.counters()
            clocks.start()
            t_ev0.record(est)
            wall0 = time.perf_counter()
        if have_kept:
            eng.draft(K_DRAFT)                    # the MTP chain: computed and timed, its tokens replaced by the scripted drafts
            if r >= a.warmup:
                dev_ms += eng.last_ms()
        drafts = [(want[done + j] + 1) % cfg.vocab if bad[r, j] else want[done + j] for j in range(K_DRAFT)]
        n, path, em = eng.verify([x] + drafts)
        if r >= a.warmup:
            dev_ms += eng.last_ms()
            tokens += n
            accepted += n - 1
            offered += K_DRAFT
        eng.commit(path)
        have_kept = True
        assert em == want[done:done + n], "speculative output diverged from the greedy continuation"
        done += n
        x = em[-1]
    t_ev1.record(est)
    barrier()
    wall = time.perf_counter() - wall0
    clk = clocks.stop()
    c1 = eng.counters()
    e2e_ms = t_ev0.elapsed_time(t_ev1)
    # max over ranks
    if world > 1:
        t = torch.tensor([dev_ms, e2e_ms], device="cuda", dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        dev_ms, e2e_ms = float(t[0]), float(t[1])
    launches = c1[0] - c0[0]
    routed_jobs_per_step = (c1[1] - c0[1]) / max(1, a.steps) if world == 1 else None
    value = tokens / (dev_ms * 1e-3)
    e2e = tokens / (e2e_ms * 1e-3)

    # ---- the verify step alone (device time of its graph), against its bytes
    vts = []
    for _ in range(5):
        eng.verify([x] + want[done:done + K_DRAFT])
        vts.append(eng.last_ms())
    verify_ms = statistics.median(vts)
    line = {"metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": dev_ms / a.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8xint3->f32",
            "data": "synthetic", "config": bench_config(workload, world, a.layers),
            "clocks": clk, "gpu_launches": int(launches),
            "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": 4 * (1 + K_DRAFT) + 4 * (1 + K_DRAFT) + 8, "d2h_bytes_per_step": 4 * 65 + 4 + 4 * K_DRAFT,
                    "wall_ms_per_step": wall * 1e3 / a.steps},
            "verify_step_us": verify_ms * 1e3, "accepted_per_offered": accepted / max(1, offered), "tokens_per_step": tokens / a.steps,
            "tokens_crc": zlib.crc32(np.asarray(want[:done], np.int64).tobytes()),
            "ep_sum": "none" if world == 1 else ("peer-memory" if use_peer else "nccl")}

    if world == 1 and rank == 0:
        import ctypes as C
        T = 1 + K_DRAFT
        # routed jobs per verify step: the counters also saw the MTP calls' routers (1 layer each, few rows); take the verify-only figure
        cA = eng.counters()
        eng.verify([x] + want[done:done + K_DRAFT])
        cB = eng.counters()
        jobs_v = cB[1] - cA[1]
        prim, allb = step_bytes(jobs_v, a.ctx + done, T)
        line["step_roofline"] = {"bound": "hbm", "primary_bytes": prim, "all_bytes": allb, "achieved_primary_gbs": prim / (verify_ms * 1e-3) / 1e9,
                                 "achieved_all_gbs": allb / (verify_ms * 1e-3) / 1e9, "peak": hbm_peak, "peak_kind": peak_kind,
                                 "frac_primary_of_measured": prim / (verify_ms * 1e-3) / 1e9 / hbm_peak,
                                 "frac_primary_of_nominal_8TBs": prim / (verify_ms * 1e-3) / 1e9 / 8000.0,
                                 "frac_all_of_measured": allb / (verify_ms * 1e-3) / 1e9 / hbm_peak, "routed_jobs": int(jobs_v)}
        # ---- the dominant kernel live: gate|up + SwiGLU of the routed experts, cycling over the 48 layers' weights
        xrow = torch.randn((T, cfg.hidden), device="cuda")
        nw = torch.ones(cfg.hidden, device="cuda")
        gu_b = F.iq3s_bytes(2 * cfg.ffn, cfg.hidden)
        routes, wgus, wshs = [], [], []
        for l in range(a.layers):
            wr = eng.tensor(f"l{l}.router", torch.float32).view(cfg.n_expert + 1, cfg.hidden)
            routes.append(F.router_route(wr, xrow, cfg.top_k, norm_w=nw))
            wgus.append(eng.tensor(f"l{l}.experts_gu", torch.uint8))
            wshs.append(eng.tensor(f"l{l}.shared_gu", torch.uint8))
        h = torch.zeros((T * cfg.top_k + T, cfg.ffn), device="cuda")
        L = F.lib()
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)

        def gate_up(l):
            r = routes[l]
            F.check(L.fnx_moe_gate_up(F.ptr(wgus[l]), gu_b, 0, F.ptr(wshs[l]), cfg.n_expert, F.ptr(r["jobs"]), F.ptr(r["njobs"]), r["njobs_max"],
                                      F.ptr(xrow), F.ptr(nw), cfg.eps, cfg.hidden, cfg.ffn, F.ptr(h), F.ptr(r["err"]), st))
        for l in range(a.layers):
            gate_up(l)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 3
        e0.record()
        for _ in range(reps):
            for l in range(a.layers):
                gate_up(l)
        e1.record()
        torch.cuda.synchronize()
        njobs = [int(r["njobs"][0].item()) for r in routes]
        per_launch_s = e0.elapsed_time(e1) * 1e-3 / (reps * a.layers)
        bytes_per_launch = sum(njobs) / len(njobs) * gu_b
        ach = bytes_per_launch / per_launch_s / 1e9
        line["roofline"] = {"bound": "hbm", "kernel": "k_iq3s_mmv<1, gate|up>", "achieved": ach, "peak": hbm_peak, "unit": "GB/s", "frac": ach / hbm_peak,
                            "peak_kind": peak_kind, "traffic": NCU_TRAFFIC_PER_JOB * sum(njobs) / len(njobs),
                            "traffic_source": "ncu dram__bytes_read+write of one gate|up launch (46 jobs, 4-layer case): 42.02 MB, scaled by jobs per launch", "us_per_launch": per_launch_s * 1e6, "jobs_per_launch": sum(njobs) / len(njobs),
                            "algorithmic_bytes_per_launch": bytes_per_launch}
        # ---- CPU restatement on the host cores, bounded sample; the full-size parity check rides along
        import oracle as O
        eng.close()
        eng = None
        cores = os.cpu_count() or 1
        samples, parity, used = cpu_leg(F, O, 2, cores)
        exp_tok = tokens / a.steps
        line["cpu_baseline"] = {"value": exp_tok / samples[-1]["step_s"], "unit": "tok/s", "cores": used, "host_cores": cores, "kind": "port",
                                "sample": CPU_SAMPLE, "extrapolated": True, "verify_step_s": samples[-1]["step_s"], "sampled_s": samples[-1]["sampled_s"]}
        line["parity_full_size"] = parity
    if eng is not None:
        eng.close()
        eng = None
    if a.layers == 48 and not a.no_config4:
        # the 8-sequence workload (configuration 4, the one expert parallelism is meant for) at this rank count, beside the headline
        import copy
        a4 = copy.copy(a)
        a4.steps, a4.warmup, a4.config = 6, 3, 4
        room = (a4.warmup + a4.steps + 8) * (K_DRAFT + 1) + 64
        cfg4 = F.flash_next_config(n_layer=48, max_ctx=C4_CTX + (room + 255) // 256 * 256, max_rows=C4_LANES * (1 + K_DRAFT), ep_rank=rank, ep_size=world, n_seq=C4_SEQS,
                                   draft_vocab=DRAFT_VOCAB)
        eng4 = F.Engine(cfg4)
        eng4.init_synthetic(seed=0, sigma=0.02)
        peer4 = ep_setup(F, eng4, rank, world)
        l4 = run_config4(a4, F, eng4, cfg4, rank, world, local, peer4, emit=False)
        line["config4"] = {k: l4[k] for k in ("value", "unit", "ms_per_step", "steps", "warmup", "verify_window_us", "tokens_per_step", "accepted_per_offered", "ep_sum",
                                             "tokens_crc", "window_bytes")}
        line["config4"]["workload"] = l4["config"]["workload"]
        line["config4"]["e2e"] = l4["e2e"]
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
