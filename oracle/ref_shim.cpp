// Reference-side half of the oracle's pins (test infrastructure only).
//
// This translation unit is compiled together with the reference's own host sources, taken from where they lie
// in the reference checkout (never copied here): engine/src/tensor_convert.hpp (header-only host dequantisers)
// and engine/src/session.cpp (make_dist, draw, lookup_drafts).  It exports a C ABI over those functions so that
// the Python tests can compare the restatement in fnx_oracle.c against the reference itself.  Built by
// oracle/Makefile into oracle/_ref/libfnx_ref.so; unused session code is dropped by --gc-sections.
#include <cstdint>
#include <utility>
#include <vector>

#include "session.hpp"
#include "tensor_convert.hpp"

#define REF_API extern "C" __attribute__((visibility("default")))

// ggml type id of IQ3_S (GGML_TYPE_IQ3_S = 21), the `type` argument of fnx::conv::dequantize
REF_API void ref_iq3s_dequant(const uint8_t* blocks, size_t nblocks, float* out) {
    fnx::conv::dequantize(fnx::T_IQ3_S, blocks, nblocks * 256, out);
}

REF_API const uint32_t* ref_iq3s_grid() { return fnx::conv::iq3s_grid(); }

REF_API uint16_t ref_f2h(float x) { return fnx::conv::f2h(x); }
REF_API float ref_h2f(uint16_t h) { return fnx::conv::h2f(h); }

static fnx::Sampling sampling(float temperature, float top_p, float min_p, int top_k) {
    fnx::Sampling s;
    s.temperature = temperature;
    s.top_p = top_p;
    s.min_p = min_p;
    s.top_k = top_k;
    return s;
}

REF_API int ref_make_dist(const float* cand_v, const int* cand_i, int n, float temperature, float top_p, float min_p,
                          int top_k, int* ids, double* p) {
    std::vector<std::pair<float, int>> cand;
    for (int i = 0; i < n; ++i) cand.emplace_back(cand_v[i], cand_i[i]);
    const fnx::Dist d = fnx::make_dist(cand, sampling(temperature, top_p, min_p, top_k));
    for (size_t i = 0; i < d.ids.size(); ++i) {
        ids[i] = d.ids[i];
        p[i] = d.p[i];
    }
    return (int) d.ids.size();
}

REF_API int ref_draw(const int* ids, const double* p, int n, double u) {
    fnx::Dist d;
    d.ids.assign(ids, ids + n);
    d.p.assign(p, p + n);
    return fnx::draw(d, u);
}

REF_API int ref_lookup(const int* ctx, int n, int lk, int d1, int* out, int* match) {
    const std::vector<int> c(ctx, ctx + n);
    const std::vector<int> r = fnx::lookup_drafts(c, lk, d1, match);
    for (size_t i = 0; i < r.size(); ++i) out[i] = r[i];
    return (int) r.size();
}
