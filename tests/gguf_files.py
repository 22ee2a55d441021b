"""GGUF files for the tests, written with gguf-py's GGUFWriter (a writer that shares no code with the reader under test).

`tiny_model_tensors` lays out a small model under llama.cpp's tensor names for this architecture from the ggml-block
bytes of an engine's own tensors, so that a second engine loaded from the file must hold the same bits."""
from __future__ import annotations

import numpy as np

ARCH = "qwen3next"


def write_gguf(path, meta: dict, tensors: dict, arch: str = ARCH):
    """meta: key (without the architecture prefix when it starts with '.') -> int | float | str | list[int];
    tensors: name -> numpy array (f32 / f16 / i32) or (bytes-shaped uint8 array, GGMLQuantizationType)."""
    import gguf
    w = gguf.GGUFWriter(str(path), arch)
    for k, v in meta.items():
        key = arch + k if k.startswith(".") else k
        if isinstance(v, bool):
            w.add_bool(key, v)
        elif isinstance(v, int):
            w.add_uint32(key, v)
        elif isinstance(v, float):
            w.add_float32(key, v)
        elif isinstance(v, str):
            w.add_string(key, v)
        else:
            w.add_array(key, list(v))
    for name, t in tensors.items():
        if isinstance(t, tuple):
            w.add_tensor(name, t[0], raw_dtype=t[1])
        else:
            w.add_tensor(name, t)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def model_meta(cfg) -> dict:
    return {
        ".block_count": cfg.n_layer + 1, ".nextn_predict_layers": 1, ".embedding_length": cfg.hidden, ".expert_count": cfg.n_expert,
        ".expert_used_count": cfg.top_k, ".expert_feed_forward_length": cfg.ffn, ".attention.head_count": cfg.n_q_head,
        ".attention.head_count_kv": cfg.n_kv_head, ".attention.key_length": cfg.head_dim, ".attention.value_length": cfg.head_dim,
        ".rope.dimension_count": cfg.n_rot, ".ssm.group_count": cfg.gdn_k_head, ".ssm.time_step_rank": cfg.gdn_v_head,
        ".ssm.state_size": cfg.gdn_head_dim, ".ssm.conv_kernel": 4, ".full_attention_interval": cfg.attn_every,
        ".attention.layer_norm_rms_epsilon": float(cfg.eps), ".rope.freq_base": float(cfg.rope_base),
    }


def tiny_model_tensors(F, eng, cfg) -> dict:
    """The engine's weights under the file's names: matrices as ggml IQ3_S blocks (un-tiled from the device), vectors f32."""
    import torch
    from gguf import GGMLQuantizationType as QT
    H, hd, hs, Fn, E = cfg.hidden, cfg.head_dim, cfg.gdn_head_dim, cfg.ffn, cfg.n_expert
    tile_rows = 16 * (16 // (H // 256))
    up = lambda v: (v + tile_rows - 1) // tile_rows * tile_rows
    out = {}

    def blocks(name, rows, cols):   # [rows][cols / 256 * 110] uint8
        t = eng.tensor(name, torch.uint8)
        return F.iq3s_untile(t, rows, cols).cpu().numpy().reshape(rows, cols // 256 * 110)

    def f32(name):
        return eng.tensor(name, torch.float32).cpu().numpy().copy()

    def layer(src, dst, attn):
        out[src + "attn_norm.weight"] = f32(dst + "norm1")
        out[src + "post_attention_norm.weight"] = f32(dst + "norm2")
        if attn:
            q, kv = cfg.n_q_head * 2 * hd, cfg.n_kv_head * hd
            w = blocks(dst + "w_in", up(q + 2 * kv), H)
            out[src + "attn_q.weight"] = (w[:q].copy(), QT.IQ3_S)
            out[src + "attn_k.weight"] = (w[q:q + kv].copy(), QT.IQ3_S)
            out[src + "attn_v.weight"] = (w[q + kv:q + 2 * kv].copy(), QT.IQ3_S)
            out[src + "attn_output.weight"] = (blocks(dst + "w_out", H, cfg.n_q_head * hd), QT.IQ3_S)
            out[src + "attn_q_norm.weight"] = f32(dst + "q_norm")
            out[src + "attn_k_norm.weight"] = f32(dst + "k_norm")
        else:
            ch, z, nv = (2 * cfg.gdn_k_head + cfg.gdn_v_head) * hs, cfg.gdn_v_head * hs, cfg.gdn_v_head
            w = blocks(dst + "w_in", up(ch + z + 2 * nv), H)
            out[src + "attn_qkv.weight"] = (w[:ch].copy(), QT.IQ3_S)
            out[src + "attn_gate.weight"] = (w[ch:ch + z].copy(), QT.IQ3_S)
            out[src + "ssm_alpha.weight"] = (w[ch + z:ch + z + nv].copy(), QT.IQ3_S)
            out[src + "ssm_beta.weight"] = (w[ch + z + nv:ch + z + 2 * nv].copy(), QT.IQ3_S)
            out[src + "ssm_out.weight"] = (blocks(dst + "w_out", H, z), QT.IQ3_S)
            out[src + "ssm_conv1d.weight"] = f32(dst + "conv_w").reshape(ch, 4)
            out[src + "ssm_dt.bias"] = f32(dst + "dt")
            out[src + "ssm_a"] = f32(dst + "a")
            out[src + "ssm_norm.weight"] = f32(dst + "g_norm")
        r = f32(dst + "router").reshape(E + 1, H)
        out[src + "ffn_gate_inp.weight"] = r[:E].copy()
        out[src + "ffn_gate_inp_shexp.weight"] = r[E].copy()
        gu = np.stack([blocks_at(F, eng, dst + "experts_gu", x, 2 * Fn, H) for x in range(E)])      # [E][2F][bytes]
        dn = np.stack([blocks_at(F, eng, dst + "experts_dn", x, H, Fn) for x in range(E)])
        out[src + "ffn_gate_exps.weight"] = (gu[:, :Fn].copy(), QT.IQ3_S)
        out[src + "ffn_up_exps.weight"] = (gu[:, Fn:].copy(), QT.IQ3_S)
        out[src + "ffn_down_exps.weight"] = (dn, QT.IQ3_S)
        sg = blocks(dst + "shared_gu", 2 * Fn, H)
        out[src + "ffn_gate_shexp.weight"] = (sg[:Fn].copy(), QT.IQ3_S)
        out[src + "ffn_up_shexp.weight"] = (sg[Fn:].copy(), QT.IQ3_S)
        out[src + "ffn_down_shexp.weight"] = (blocks(dst + "shared_dn", H, Fn), QT.IQ3_S)

    for l in range(cfg.n_layer):
        layer(f"blk.{l}.", f"l{l}.", (l + 1) % cfg.attn_every == 0)
    m = f"blk.{cfg.n_layer}."
    layer(m, "mtp.", True)
    out[m + "nextn.enorm.weight"] = f32("mtp.e_norm")
    out[m + "nextn.hnorm.weight"] = f32("mtp.h_norm")
    out[m + "nextn.shared_head_norm.weight"] = f32("mtp.out_norm")
    out[m + "nextn.eh_proj.weight"] = (np.concatenate([blocks("mtp.fc_emb", H, H), blocks("mtp.fc_hid", H, H)], axis=1), QT.IQ3_S)
    out["output_norm.weight"] = f32("out_norm")
    out["output.weight"] = (blocks("head", cfg.vocab, H), QT.IQ3_S)
    if cfg.draft_vocab:
        out[m + "nextn.shared_head_head.weight"] = (blocks("mtp.head", cfg.draft_vocab, H), QT.IQ3_S)
        out[m + "nextn.draft_vocab"] = eng.tensor("mtp.vocab", torch.int32).cpu().numpy().copy()
    out["token_embd.weight"] = eng.tensor("embed", torch.float16).cpu().numpy().reshape(cfg.vocab, H).copy()
    return out


def blocks_at(F, eng, name, x, rows, cols):
    """ggml blocks of expert x of a stacked expert tensor of the engine"""
    import torch
    per = F.iq3s_bytes(rows, cols)
    t = eng.tensor(name, torch.uint8)[x * per:(x + 1) * per]
    return F.iq3s_untile(t, rows, cols).cpu().numpy().reshape(rows, cols // 256 * 110)
