// Model loader: a GGUF file's tensors (llama.cpp's names for this architecture) into an engine's device tensors.  The
// counterpart of the reference's load (engine/src/model.cpp:837-905 dense models, :932-1097 the MoE model; expert slicing
// :1063-1069; small-tensor conversion engine/src/tensor_convert.hpp): every matrix ends up in the IQ3_S tile layout the
// kernels stream, every vector in f32.
//   - an IQ3_S tensor is copied block for block and re-tiled: bit-exact;
//   - a matrix of another type (F32, F16, BF16, Q8_0) is converted to f32 on the host and quantised to IQ3_S on the
//     GPU by fnx_iq3s_quantize: lossy, counted in *h_converted (the verify path has no kernels for other formats);
//   - stacked expert tensors ([experts][rows][cols]) are sliced to this rank's experts.
// Written against the public entry points only (fnx_engine_tensor names the destinations).
#include <cstring>
#include <string>
#include <vector>

#include "fnx_common.cuh"

namespace fnxb {

namespace {

constexpr size_t IQ3S_BLOCK = 110;

struct Piece {
    fnx_gguf_tensor t;
    int64_t row0, n_rows;     // rows of the source (a row = ne[0] weights)
    int64_t col0, n_cols;     // columns of the source, whole 256-weight blocks
};

struct Loader {
    fnx_engine* e;
    const fnx_gguf* g;
    fnx_model_config c;
    cudaStream_t st;
    int converted = 0;
    float* d_f = nullptr;        // staging: f32 weights of one chunk
    uint8_t* d_g = nullptr;      // staging: GGML blocks of one destination matrix
    size_t f_cap = 0, g_cap = 0;
    std::vector<float> h_f;

    ~Loader() {
        if (d_f) cudaFree(d_f);
        if (d_g) cudaFree(d_g);
    }

    int find(const std::string& name, fnx_gguf_tensor* t) const {
        if (!fnx_gguf_find(g, name.c_str(), t)) return fail(FNX_E_ARG, "load: the file has no tensor %s", name.c_str());
        return FNX_OK;
    }

    int dest(const std::string& name, size_t want_bytes, void** p) const {
        size_t bytes = 0;
        *p = fnx_engine_tensor(e, name.c_str(), &bytes);
        if (!*p) return fail(FNX_E_STATE, "load: the engine has no tensor %s", name.c_str());
        if (bytes != want_bytes) return fail(FNX_E_STATE, "load: engine tensor %s holds %zu bytes, the loader fills %zu", name.c_str(), bytes, want_bytes);
        return FNX_OK;
    }

    int need_g(size_t bytes) {
        if (bytes <= g_cap) return FNX_OK;
        if (d_g) cudaFree(d_g);
        d_g = nullptr;
        g_cap = 0;
        FNX_CUDA_OK(cudaMalloc((void**) &d_g, bytes));
        g_cap = bytes;
        return FNX_OK;
    }

    int need_f(size_t floats) {
        if (floats <= f_cap) return FNX_OK;
        if (d_f) cudaFree(d_f);
        d_f = nullptr;
        f_cap = 0;
        FNX_CUDA_OK(cudaMalloc((void**) &d_f, floats * sizeof(float)));
        f_cap = floats;
        return FNX_OK;
    }

    // A matrix of `rows` x `cols` from pieces stacked by rows, in order; rows past the pieces' are zero.  Every piece has
    // `cols` columns (n_cols) and its rows land after the previous piece's.
    int matrix(const std::string& dst_name, size_t rows, size_t cols, const std::vector<Piece>& pieces) {
        void* dst = nullptr;
        FNX_TRY(dest(dst_name, fnx_iq3s_bytes(rows, cols), &dst));
        return matrix_to(dst, dst_name, rows, cols, pieces);
    }

    int matrix_to(void* dst, const std::string& what, size_t rows, size_t cols, const std::vector<Piece>& pieces) {
        FNX_REQUIRE(rows % 16 == 0 && cols % 256 == 0, "load: %s is %zu x %zu (rows in 16s, columns in 256s)", what.c_str(), rows, cols);
        const size_t row_bytes = cols / 256 * IQ3S_BLOCK;
        FNX_TRY(need_g(rows * row_bytes));
        FNX_CUDA_OK(cudaMemsetAsync(d_g, 0, rows * row_bytes, st));
        size_t r = 0;
        for (const Piece& p : pieces) {
            FNX_REQUIRE((size_t) p.n_cols == cols && p.col0 % 256 == 0, "load: %s: a piece of %s has %lld columns from %lld, the matrix %zu", what.c_str(),
                        p.t.name, (long long) p.n_cols, (long long) p.col0, cols);
            FNX_REQUIRE(p.row0 >= 0 && p.col0 + p.n_cols <= p.t.ne[0] && p.row0 + p.n_rows <= p.t.ne[1] * p.t.ne[2] * p.t.ne[3],
                        "load: %s: rows [%lld, %lld) x columns [%lld, %lld) are not inside %s", what.c_str(), (long long) p.row0,
                        (long long) (p.row0 + p.n_rows), (long long) p.col0, (long long) (p.col0 + p.n_cols), p.t.name);
            FNX_REQUIRE(r + (size_t) p.n_rows <= rows, "load: %s: more rows in the file than the matrix has (%zu)", what.c_str(), rows);
            uint8_t* at = d_g + r * row_bytes;
            if (p.t.type == 21) {   // IQ3_S: the blocks as they are
                const size_t src_row = (size_t) p.t.ne[0] / 256 * IQ3S_BLOCK;
                const uint8_t* src = (const uint8_t*) p.t.data + (size_t) p.row0 * src_row + (size_t) p.col0 / 256 * IQ3S_BLOCK;
                FNX_CUDA_OK(cudaMemcpy2DAsync(at, row_bytes, src, src_row, row_bytes, (size_t) p.n_rows, cudaMemcpyHostToDevice, st));
            } else {   // another type: f32 on the host, IQ3_S on the GPU
                const size_t chunk_rows = ((size_t) 8 << 20) / cols ? ((size_t) 8 << 20) / cols : 1;
                for (size_t r0 = 0; r0 < (size_t) p.n_rows; r0 += chunk_rows) {
                    const size_t nr = (size_t) p.n_rows - r0 < chunk_rows ? (size_t) p.n_rows - r0 : chunk_rows;
                    h_f.resize(nr * (size_t) p.t.ne[0]);
                    FNX_TRY(fnx_gguf_rows_f32(&p.t, p.row0 + (int64_t) r0, (int64_t) nr, h_f.data()));
                    FNX_TRY(need_f(nr * cols));
                    FNX_CUDA_OK(cudaMemcpy2DAsync(d_f, cols * sizeof(float), h_f.data() + p.col0, (size_t) p.t.ne[0] * sizeof(float), cols * sizeof(float), nr,
                                                  cudaMemcpyHostToDevice, st));
                    FNX_TRY(fnx_iq3s_quantize(d_f, at + r0 * row_bytes, nr * cols, st));
                    FNX_CUDA_OK(cudaStreamSynchronize(st));   // h_f is reused by the next chunk
                }
                ++converted;
            }
            r += (size_t) p.n_rows;
        }
        FNX_TRY(fnx_iq3s_retile(d_g, dst, rows, cols, st));
        FNX_CUDA_OK(cudaStreamSynchronize(st));
        return FNX_OK;
    }

    Piece whole(const fnx_gguf_tensor& t) const { return Piece{t, 0, t.ne[1] * t.ne[2] * t.ne[3], 0, t.ne[0]}; }

    // an f32 vector (or small f32 table) of n values from a tensor of any convertible type
    int vec(const std::string& dst_name, const std::string& src_name, size_t n) {
        fnx_gguf_tensor t;
        FNX_TRY(find(src_name, &t));
        const size_t have = (size_t) (t.ne[0] * t.ne[1] * t.ne[2] * t.ne[3]);
        FNX_REQUIRE(have == n, "load: %s holds %zu values, %s takes %zu", src_name.c_str(), have, dst_name.c_str(), n);
        void* dst = nullptr;
        FNX_TRY(dest(dst_name, n * sizeof(float), &dst));
        h_f.resize(n);
        FNX_TRY(fnx_gguf_rows_f32(&t, 0, t.ne[1] * t.ne[2] * t.ne[3], h_f.data()));
        FNX_CUDA_OK(cudaMemcpyAsync(dst, h_f.data(), n * sizeof(float), cudaMemcpyHostToDevice, st));
        FNX_CUDA_OK(cudaStreamSynchronize(st));
        return FNX_OK;
    }

    int mixer_and_experts(int l, bool attn, const std::string& src, const std::string& dst) {
        const int H = c.hidden, hd = c.head_dim, hs = c.gdn_head_dim;
        const size_t tile_rows = (size_t) 16 * (16 / (H / 256));
        auto round_up = [&](size_t v) { return (v + tile_rows - 1) / tile_rows * tile_rows; };
        fnx_gguf_tensor a, b, d3, d4;
        FNX_TRY(vec(dst + "norm1", src + "attn_norm.weight", (size_t) H));
        FNX_TRY(vec(dst + "norm2", src + "post_attention_norm.weight", (size_t) H));
        if (attn) {
            // rows: every query head's q | gate (attn_q.weight holds both), then the key heads, then the value heads
            const size_t q_rows = (size_t) c.n_q_head * 2 * hd, kv_rows = (size_t) c.n_kv_head * hd;
            FNX_TRY(find(src + "attn_q.weight", &a));
            FNX_TRY(find(src + "attn_k.weight", &b));
            FNX_TRY(find(src + "attn_v.weight", &d3));
            FNX_REQUIRE((size_t) a.ne[1] == q_rows && (size_t) b.ne[1] == kv_rows && (size_t) d3.ne[1] == kv_rows, "load: layer %d: q | k | v of %lld, %lld, %lld rows (%zu, %zu, %zu)",
                        l, (long long) a.ne[1], (long long) b.ne[1], (long long) d3.ne[1], q_rows, kv_rows, kv_rows);
            FNX_TRY(matrix(dst + "w_in", round_up(q_rows + 2 * kv_rows), (size_t) H, {whole(a), whole(b), whole(d3)}));
            FNX_TRY(find(src + "attn_output.weight", &a));
            FNX_TRY(matrix(dst + "w_out", (size_t) H, (size_t) c.n_q_head * hd, {whole(a)}));
            FNX_TRY(vec(dst + "q_norm", src + "attn_q_norm.weight", (size_t) hd));
            FNX_TRY(vec(dst + "k_norm", src + "attn_k_norm.weight", (size_t) hd));
        } else {
            // rows: the conv channels q | k | v (attn_qkv.weight), the output gate z (attn_gate.weight), alpha, beta
            const size_t ch = (size_t) (2 * c.gdn_k_head + c.gdn_v_head) * hs, z = (size_t) c.gdn_v_head * hs, nv = (size_t) c.gdn_v_head;
            FNX_TRY(find(src + "attn_qkv.weight", &a));
            FNX_TRY(find(src + "attn_gate.weight", &b));
            FNX_TRY(find(src + "ssm_alpha.weight", &d3));
            FNX_TRY(find(src + "ssm_beta.weight", &d4));
            FNX_REQUIRE((size_t) a.ne[1] == ch && (size_t) b.ne[1] == z && (size_t) d3.ne[1] == nv && (size_t) d4.ne[1] == nv,
                        "load: layer %d: qkv | gate | alpha | beta of %lld, %lld, %lld, %lld rows (%zu, %zu, %zu, %zu)", l, (long long) a.ne[1], (long long) b.ne[1],
                        (long long) d3.ne[1], (long long) d4.ne[1], ch, z, nv, nv);
            FNX_TRY(matrix(dst + "w_in", round_up(ch + z + 2 * nv), (size_t) H, {whole(a), whole(b), whole(d3), whole(d4)}));
            FNX_TRY(find(src + "ssm_out.weight", &a));
            FNX_TRY(matrix(dst + "w_out", (size_t) H, z, {whole(a)}));
            FNX_TRY(vec(dst + "conv_w", src + "ssm_conv1d.weight", ch * 4));
            FNX_TRY(vec(dst + "dt", src + "ssm_dt.bias", nv));
            FNX_TRY(vec(dst + "a", src + "ssm_a", nv));
            FNX_TRY(vec(dst + "g_norm", src + "ssm_norm.weight", (size_t) hs));
        }
        // router rows: the experts' (ffn_gate_inp.weight), then the shared expert's gate (ffn_gate_inp_shexp.weight)
        {
            fnx_gguf_tensor r, s;
            FNX_TRY(find(src + "ffn_gate_inp.weight", &r));
            FNX_TRY(find(src + "ffn_gate_inp_shexp.weight", &s));
            FNX_REQUIRE(r.ne[0] == H && r.ne[1] == c.n_expert && s.ne[0] * s.ne[1] == H, "load: layer %d: router of %lld x %lld, shared gate of %lld", l,
                        (long long) r.ne[1], (long long) r.ne[0], (long long) (s.ne[0] * s.ne[1]));
            void* wr = nullptr;
            FNX_TRY(dest(dst + "router", (size_t) (c.n_expert + 1) * H * sizeof(float), &wr));
            h_f.resize((size_t) (c.n_expert + 1) * H);
            FNX_TRY(fnx_gguf_rows_f32(&r, 0, c.n_expert, h_f.data()));
            FNX_TRY(fnx_gguf_rows_f32(&s, 0, s.ne[1], h_f.data() + (size_t) c.n_expert * H));
            FNX_CUDA_OK(cudaMemcpyAsync(wr, h_f.data(), h_f.size() * sizeof(float), cudaMemcpyHostToDevice, st));
            FNX_CUDA_OK(cudaStreamSynchronize(st));
        }
        // this rank's experts: gate rows then up rows per expert; down
        const int F = c.ffn, E_local = c.n_expert / c.ep_size, e_lo = c.ep_rank * E_local;
        fnx_gguf_tensor tg, tu, td;
        FNX_TRY(find(src + "ffn_gate_exps.weight", &tg));
        FNX_TRY(find(src + "ffn_up_exps.weight", &tu));
        FNX_TRY(find(src + "ffn_down_exps.weight", &td));
        FNX_REQUIRE(tg.ne[0] == H && tg.ne[1] == F && tg.ne[2] == c.n_expert && tu.ne[0] == H && tu.ne[1] == F && tu.ne[2] == c.n_expert && td.ne[0] == F &&
                        td.ne[1] == H && td.ne[2] == c.n_expert,
                    "load: layer %d: the stacked expert tensors are not [%d][%d][%d] (gate, up) and [%d][%d][%d] (down)", l, c.n_expert, F, H, c.n_expert, H, F);
        const size_t gu_bytes = fnx_iq3s_bytes((size_t) 2 * F, (size_t) H), dn_bytes = fnx_iq3s_bytes((size_t) H, (size_t) F);
        void *wgu = nullptr, *wdn = nullptr;
        FNX_TRY(dest(dst + "experts_gu", gu_bytes * E_local, &wgu));
        FNX_TRY(dest(dst + "experts_dn", dn_bytes * E_local, &wdn));
        const int conv0 = converted;
        for (int x = 0; x < E_local; ++x) {
            const int64_t ge = e_lo + x;
            FNX_TRY(matrix_to((uint8_t*) wgu + (size_t) x * gu_bytes, dst + "experts_gu", (size_t) 2 * F, (size_t) H,
                              {Piece{tg, ge * F, F, 0, H}, Piece{tu, ge * F, F, 0, H}}));
            FNX_TRY(matrix_to((uint8_t*) wdn + (size_t) x * dn_bytes, dst + "experts_dn", (size_t) H, (size_t) F, {Piece{td, ge * H, H, 0, F}}));
        }
        if (converted > conv0) converted = conv0 + (tg.type != 21) + (tu.type != 21) + (td.type != 21);   // counted per tensor, not per expert
        FNX_TRY(find(src + "ffn_gate_shexp.weight", &tg));
        FNX_TRY(find(src + "ffn_up_shexp.weight", &tu));
        FNX_TRY(find(src + "ffn_down_shexp.weight", &td));
        FNX_TRY(matrix(dst + "shared_gu", (size_t) 2 * F, (size_t) H, {whole(tg), whole(tu)}));
        FNX_TRY(matrix(dst + "shared_dn", (size_t) H, (size_t) F, {whole(td)}));
        return FNX_OK;
    }

    int run() {
        const int H = c.hidden, NL = c.n_layer;
        for (int l = 0; l < NL; ++l)
            FNX_TRY(mixer_and_experts(l, (l + 1) % c.attn_every == 0, "blk." + std::to_string(l) + ".", "l" + std::to_string(l) + "."));
        // the next-token layer: block NL of the file, an attention layer, with its own input projections and norms
        const std::string m = "blk." + std::to_string(NL) + ".";
        FNX_TRY(mixer_and_experts(NL, true, m, "mtp."));
        FNX_TRY(vec("mtp.e_norm", m + "nextn.enorm.weight", (size_t) H));
        FNX_TRY(vec("mtp.h_norm", m + "nextn.hnorm.weight", (size_t) H));
        FNX_TRY(vec("mtp.out_norm", m + "nextn.shared_head_norm.weight", (size_t) H));
        {   // eh_proj [H][2 H]: columns [0, H) multiply the normed embedding, [H, 2 H) the normed hidden row
            fnx_gguf_tensor eh;
            FNX_TRY(find(m + "nextn.eh_proj.weight", &eh));
            FNX_REQUIRE(eh.ne[0] == 2 * H && eh.ne[1] == H, "load: %snextn.eh_proj.weight is %lld x %lld, not %d x %d", m.c_str(), (long long) eh.ne[1],
                        (long long) eh.ne[0], H, 2 * H);
            FNX_TRY(matrix("mtp.fc_emb", (size_t) H, (size_t) H, {Piece{eh, 0, H, 0, H}}));
            FNX_TRY(matrix("mtp.fc_hid", (size_t) H, (size_t) H, {Piece{eh, 0, H, H, H}}));
        }
        FNX_TRY(vec("out_norm", "output_norm.weight", (size_t) H));
        fnx_gguf_tensor t;
        FNX_TRY(find("output.weight", &t));
        FNX_REQUIRE(t.ne[0] == H && t.ne[1] == c.vocab, "load: output.weight is %lld x %lld, not %d x %d", (long long) t.ne[1], (long long) t.ne[0], c.vocab, H);
        FNX_TRY(matrix("head", (size_t) c.vocab, (size_t) H, {whole(t)}));
        if (c.draft_vocab > 0) {   // the draft layer's own head and the token id of each of its rows
            FNX_TRY(find(m + "nextn.shared_head_head.weight", &t));
            FNX_REQUIRE(t.ne[0] == H && t.ne[1] == c.draft_vocab, "load: the draft head is %lld x %lld, not %d x %d", (long long) t.ne[1], (long long) t.ne[0],
                        c.draft_vocab, H);
            FNX_TRY(matrix("mtp.head", (size_t) c.draft_vocab, (size_t) H, {whole(t)}));
            FNX_TRY(find(m + "nextn.draft_vocab", &t));
            FNX_REQUIRE(t.type == 26 && t.ne[0] == c.draft_vocab, "load: %snextn.draft_vocab is not %d I32 token ids", m.c_str(), c.draft_vocab);
            const int32_t* ids = (const int32_t*) t.data;
            for (int i = 0; i < c.draft_vocab; ++i) FNX_REQUIRE(ids[i] >= 0 && ids[i] < c.vocab, "load: draft vocabulary row %d is token %d", i, ids[i]);
            void* dv = nullptr;
            FNX_TRY(dest("mtp.vocab", (size_t) c.draft_vocab * sizeof(int), &dv));
            FNX_CUDA_OK(cudaMemcpyAsync(dv, ids, (size_t) c.draft_vocab * sizeof(int), cudaMemcpyHostToDevice, st));
            FNX_CUDA_OK(cudaStreamSynchronize(st));
        }
        // the embedding table in f16, a chunk of rows at a time
        FNX_TRY(find("token_embd.weight", &t));
        FNX_REQUIRE(t.ne[0] == H && t.ne[1] == c.vocab, "load: token_embd.weight is %lld x %lld, not %d x %d", (long long) t.ne[1], (long long) t.ne[0], c.vocab, H);
        void* emb = nullptr;
        FNX_TRY(dest("embed", (size_t) c.vocab * H * sizeof(__half), &emb));
        if (t.type == 1) {
            FNX_CUDA_OK(cudaMemcpyAsync(emb, t.data, (size_t) c.vocab * H * sizeof(__half), cudaMemcpyHostToDevice, st));
            FNX_CUDA_OK(cudaStreamSynchronize(st));
        } else {
            const size_t chunk = 4096;
            std::vector<__half> hh;
            for (size_t r0 = 0; r0 < (size_t) c.vocab; r0 += chunk) {
                const size_t nr = (size_t) c.vocab - r0 < chunk ? (size_t) c.vocab - r0 : chunk;
                h_f.resize(nr * H);
                hh.resize(nr * H);
                FNX_TRY(fnx_gguf_rows_f32(&t, (int64_t) r0, (int64_t) nr, h_f.data()));
                for (size_t i = 0; i < nr * (size_t) H; ++i) hh[i] = __float2half_rn(h_f[i]);
                FNX_CUDA_OK(cudaMemcpyAsync((__half*) emb + r0 * H, hh.data(), nr * H * sizeof(__half), cudaMemcpyHostToDevice, st));
                FNX_CUDA_OK(cudaStreamSynchronize(st));
            }
        }
        return FNX_OK;
    }
};

}  // namespace

}  // namespace fnxb

using namespace fnxb;

extern "C" int fnx_engine_load_gguf(fnx_engine* e, const fnx_gguf* g, int* h_converted) {
    FNX_REQUIRE(e && g, "fnx_engine_load_gguf: null argument");
    if (h_converted) *h_converted = 0;
    Loader L;
    L.e = e;
    L.g = g;
    FNX_TRY(fnx_engine_config(e, &L.c));
    fnx_model_config f = L.c;
    FNX_TRY(fnx_gguf_model_config(g, &f));
    const fnx_model_config& c = L.c;
    FNX_REQUIRE(f.n_layer == c.n_layer && f.hidden == c.hidden && f.n_expert == c.n_expert && f.top_k == c.top_k && f.ffn == c.ffn && f.n_q_head == c.n_q_head &&
                    f.n_kv_head == c.n_kv_head && f.head_dim == c.head_dim && f.n_rot == c.n_rot && f.gdn_k_head == c.gdn_k_head && f.gdn_v_head == c.gdn_v_head &&
                    f.gdn_head_dim == c.gdn_head_dim && f.vocab == c.vocab && f.attn_every == c.attn_every && f.draft_vocab == c.draft_vocab,
                "fnx_engine_load_gguf: the file's architecture is not the engine's (make the engine from fnx_gguf_model_config)");
    L.st = (cudaStream_t) fnx_engine_stream(e);
    const int rc = L.run();
    if (h_converted) *h_converted = L.converted;
    return rc;
}
