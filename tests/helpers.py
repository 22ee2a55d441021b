"""Shared pieces of the GPU parity tests: weight fixtures and the oracle-side model."""
from __future__ import annotations

import numpy as np


def gpu_iq3s_matrix(F, rows, cols, seed, stream_id, sigma=0.02):
    """A random IQ3_S matrix made on the GPU: returns (tiles cuda uint8, ggml bytes numpy)."""
    import torch
    w = torch.empty(rows * cols, dtype=torch.float32, device="cuda")
    F.fill_normal(w, sigma, seed, stream_id)
    g = F.iq3s_quantize(w)
    t = F.iq3s_retile(g, rows, cols)
    return t, g.cpu().numpy()


def rel_err(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


class OracleModel:
    """The synthetic model run through the CPU oracle, on the weights the engine holds.

    Mirrors the engine's data flow (engine.cu: enqueue_verify / enqueue_mtp): pre-norm residual blocks, the input
    projection rows laid out [q|gate per head; k; v] or [q|k|v|z|alpha|beta], ring slots for the DeltaNet state."""

    def __init__(self, F, O, eng, cfg, layers=None, with_mtp=True):
        import torch
        self.O, self.cfg = O, cfg
        c = cfg
        self.H, self.E, self.K, self.Fn = c.hidden, c.n_expert, c.top_k, c.ffn
        self.nq, self.nkv, self.hd, self.nrot = c.n_q_head, c.n_kv_head, c.head_dim, c.n_rot
        self.nk, self.nv, self.hs, self.V = c.gdn_k_head, c.gdn_v_head, c.gdn_head_dim, c.vocab
        self.NS = c.max_rows + 1
        self.cache_rows = c.max_ctx + c.max_rows
        tile_rows = 16 * (16 // (c.hidden // 256))
        up = lambda v: (v + tile_rows - 1) // tile_rows * tile_rows
        self.q_rows, self.kv_rows = self.nq * 2 * self.hd, self.nkv * self.hd
        self.attn_in = up(self.q_rows + 2 * self.kv_rows)
        self.ch = (2 * self.nk + self.nv) * self.hs
        self.gdn_in = up(self.ch + self.nv * self.hs + 2 * self.nv)

        def f32(name):
            return eng.tensor(name, torch.float32).cpu().numpy().copy()

        def iq(name, rows, cols):
            t = eng.tensor(name, torch.uint8)
            return F.iq3s_untile(t, rows, cols).cpu().numpy()

        def layer(pre, attn):
            L = dict(attn=attn, norm1=f32(pre + "norm1"), norm2=f32(pre + "norm2"))
            if attn:
                L["w_in"] = iq(pre + "w_in", self.attn_in, self.H)
                L["w_out"] = iq(pre + "w_out", self.H, self.nq * self.hd)
                L["qn"], L["kn"] = f32(pre + "q_norm"), f32(pre + "k_norm")
                L["kc"] = np.zeros((self.cache_rows, self.nkv, self.hd), np.uint16)
                L["vc"] = np.zeros((self.cache_rows, self.nkv, self.hd), np.uint16)
            else:
                L["w_in"] = iq(pre + "w_in", self.gdn_in, self.H)
                L["w_out"] = iq(pre + "w_out", self.H, self.nv * self.hs)
                L["convw"], L["dt"], L["a"], L["gnorm"] = f32(pre + "conv_w"), f32(pre + "dt"), f32(pre + "a"), f32(pre + "g_norm")
                L["S"] = np.zeros((self.NS, self.nv, self.hs, self.hs), np.float32)
                L["hist"] = np.zeros((self.NS, 3, self.ch), np.float32)
            L["wr"] = f32(pre + "router").reshape(self.E + 1, self.H)
            gu_b, dn_b = 2 * self.Fn * (self.H // 256) * 110, self.H * (self.Fn // 256) * 110
            gu = eng.tensor(pre + "experts_gu", torch.uint8)
            dn = eng.tensor(pre + "experts_dn", torch.uint8)
            L["wgu"] = np.concatenate([F.iq3s_untile(gu[i * gu_b:(i + 1) * gu_b], 2 * self.Fn, self.H).cpu().numpy() for i in range(self.E)])
            L["wdn"] = np.concatenate([F.iq3s_untile(dn[i * dn_b:(i + 1) * dn_b], self.H, self.Fn).cpu().numpy() for i in range(self.E)])
            L["wsh_gu"] = iq(pre + "shared_gu", 2 * self.Fn, self.H)
            L["wsh_dn"] = iq(pre + "shared_dn", self.H, self.Fn)
            return L

        ids = range(c.n_layer) if layers is None else layers
        self.layers = [layer(f"l{l}.", (l + 1) % c.attn_every == 0) for l in ids]
        self.mtp = layer("mtp.", True) if with_mtp else None
        self.mtp_hnorm, self.mtp_enorm, self.mtp_onorm = f32("mtp.h_norm"), f32("mtp.e_norm"), f32("mtp.out_norm")
        self.out_norm = f32("out_norm")
        self.fc_hid, self.fc_emb = iq("mtp.fc_hid", self.H, self.H), iq("mtp.fc_emb", self.H, self.H)
        self.head = iq("head", self.V, self.H)
        # the draft layer's own head over a draft vocabulary (head row -> token id), or the main head
        self.dvn = int(getattr(c, "draft_vocab", 0)) or self.V
        self.mtp_head, self.dvocab = self.head, None
        if with_mtp and self.dvn != self.V:
            self.mtp_head = iq("mtp.head", self.dvn, self.H)
            self.dvocab = eng.tensor("mtp.vocab", torch.int32).cpu().numpy().copy()
        self.embed = eng.tensor("embed", torch.float16).cpu().numpy().reshape(self.V, self.H).astype(np.float32)
        self.pos, self.cur = 0, 0
        self.routing = []

    # ---- blocks
    def _attention(self, L, R, pos0, parent, depth):
        O, T = self.O, R.shape[0]
        y = O.iq3s_gemv(L["w_in"], self.attn_in, self.H, O.rmsnorm(R, L["norm1"], self.cfg.eps))
        qg = np.ascontiguousarray(y[:, :self.q_rows]).reshape(T, self.nq, 2 * self.hd)
        k = np.ascontiguousarray(y[:, self.q_rows:self.q_rows + self.kv_rows]).reshape(T, self.nkv, self.hd)
        v = np.ascontiguousarray(y[:, self.q_rows + self.kv_rows:self.q_rows + 2 * self.kv_rows]).reshape(T, self.nkv, self.hd)
        O.attn_prep_append(qg, k, v, L["qn"], L["kn"], L["kc"], L["vc"], pos0, depth, self.nrot, self.cfg.eps, self.cfg.rope_base)
        out = O.attn(qg, L["kc"], L["vc"], pos0, parent).reshape(T, self.nq * self.hd)
        return R + O.iq3s_gemv(L["w_out"], self.H, self.nq * self.hd, out)

    def _gdn(self, L, R, parent):
        O, T = self.O, R.shape[0]
        y = O.iq3s_gemv(L["w_in"], self.gdn_in, self.H, O.rmsnorm(R, L["norm1"], self.cfg.eps))
        w = self.ch + self.nv * self.hs
        qkvz = np.ascontiguousarray(y[:, :w])
        ab = np.ascontiguousarray(y[:, w:w + 2 * self.nv])
        out = O.gdn_core(qkvz, ab, L["hist"], L["convw"], L["dt"], L["a"], L["gnorm"], L["S"], self.cur, parent, self.nk, self.nv, self.hs,
                         self.cfg.eps)
        return R + O.iq3s_gemv(L["w_out"], self.H, self.nv * self.hs, out)

    def _moe(self, L, R):
        O = self.O
        out, logits, topi, topw = O.moe(L["wr"], L["wgu"], L["wdn"], L["wsh_gu"], L["wsh_dn"], O.rmsnorm(R, L["norm2"], self.cfg.eps), self.Fn,
                                        self.K)
        self.routing.append((topi.copy(), logits.copy()))
        return R + out

    def verify(self, tokens, parent=None):
        O, T = self.O, len(tokens)
        depth = None
        if parent is not None:
            depth = [0] * T
            for t in range(1, T):
                depth[t] = depth[parent[t]] + 1
        R = self.embed[np.asarray(tokens)].copy()
        self.routing = []
        for L in self.layers:
            R = self._attention(L, R, self.pos, parent, depth) if L["attn"] else self._gdn(L, R, parent)
            R = self._moe(L, R)
        self.R = R
        self.tok, self.parent = list(tokens), parent
        self.logits = O.iq3s_gemv(self.head, self.V, self.H, O.rmsnorm(R, self.out_norm, self.cfg.eps))
        self.best, _ = O.argmax(self.logits)
        return O.accept_greedy(tokens, parent, self.best)

    def commit(self, path):
        path = [int(v) for v in path]
        n = len(path)
        for L in self.layers:
            if L["attn"]:
                for j, s in enumerate(path):
                    if s != j:
                        L["kc"][self.pos + j] = L["kc"][self.pos + s]
                        L["vc"][self.pos + j] = L["vc"][self.pos + s]
        self.kept_rows = self.R[np.asarray(path)].copy()
        self.kept_pos0 = self.pos
        self.cur = int((self.cur + 1 + int(path[-1])) % self.NS)
        self.pos += n

    def _mtp_call(self, src, toks, pos0):
        O = self.O
        emb = self.embed[np.asarray(toks)]
        Rm = O.iq3s_gemv(self.fc_hid, self.H, self.H, O.rmsnorm(src, self.mtp_hnorm, self.cfg.eps)) + \
            O.iq3s_gemv(self.fc_emb, self.H, self.H, O.rmsnorm(emb, self.mtp_enorm, self.cfg.eps))
        Rm = self._attention(self.mtp, Rm, pos0, None, None)
        Rm = self._moe(self.mtp, Rm)
        logits = O.iq3s_gemv(self.mtp_head, self.dvn, self.H, O.rmsnorm(Rm[-1:], self.mtp_onorm, self.cfg.eps))
        row = int(O.argmax(logits)[0][0])
        return Rm, row if self.dvocab is None else int(self.dvocab[row])

    def draft(self, emitted, k):
        n = len(emitted)
        Rm, d = self._mtp_call(self.kept_rows, emitted, self.kept_pos0)
        out = [d]
        for j in range(1, k):
            src = Rm[n - 1:n] if j == 1 else Rm[0:1]
            Rm, d = self._mtp_call(src, [out[-1]], self.kept_pos0 + n - 1 + j)
            out.append(d)
        return out
