// Load-time work on IQ3_S weights: GGML blocks <-> device tiles, tiles -> f32, the fixture quantiser and the
// Philox normal generator that makes synthetic weights.
//
// The reference's counterparts are host code: the per-card slicing and re-layout of the loader
// (engine/src/model.cpp:1063-1069, the split Q8_0 layout of engine/src/dense.cuh) and the host dequantiser
// (engine/src/tensor_convert.hpp:295-322).  Here they run on the GPU because a 48-layer synthetic model is
// 79 G weights.
#include "fnx_common.cuh"
#include "iq3s_grid.h"
#include "iq3s_tile.h"

namespace fnxb {

__device__ const uint32_t g_grid_prep[512] = {FNX_IQ3S_GRID_VALUES};

// one thread per (tile, row): rows * K/256 blocks in all
__global__ void k_retile(const uint8_t* __restrict__ ggml, uint8_t* __restrict__ tiles, size_t rows, int KB, int inverse) {
    const size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * KB) return;
    const size_t row = i / KB;
    const int b = (int) (i % KB);
    uint8_t* tile = tiles + ((row / 16) * KB + b) * TILE_BYTES;
    uint8_t blk[IQ3S_BLOCK_BYTES];
    if (!inverse) {
        const uint8_t* src = ggml + (row * KB + b) * IQ3S_BLOCK_BYTES;
        for (int k = 0; k < IQ3S_BLOCK_BYTES; ++k) blk[k] = src[k];
        tile_put_block(tile, (int) (row % 16), blk);
    } else {
        tile_get_block(tile, (int) (row % 16), blk);
        uint8_t* dst = const_cast<uint8_t*>(ggml) + (row * KB + b) * IQ3S_BLOCK_BYTES;
        for (int k = 0; k < IQ3S_BLOCK_BYTES; ++k) dst[k] = blk[k];
    }
}

// tiles -> f32 [rows][cols]: value = (d (1 + 2 s)) * g * sign, the order of the reference's host dequantiser
__global__ void k_dequant_tiles(const uint8_t* __restrict__ tiles, float* __restrict__ out, size_t rows, int KB) {
    const size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * KB) return;
    const size_t row = i / KB;
    const int b = (int) (i % KB);
    uint8_t blk[IQ3S_BLOCK_BYTES];
    tile_get_block(tiles + ((row / 16) * KB + b) * TILE_BYTES, (int) (row % 16), blk);
    const float d = __half2float(__ushort_as_half((unsigned short) (blk[0] | (blk[1] << 8))));
    const uint8_t *qs = blk + 2, *qh = blk + 66, *signs = blk + 74, *scales = blk + 106;
    float* o = out + (row * KB + b) * 256;
    for (int ib = 0; ib < 8; ++ib) {
        const float db = __fmul_rn(d, (float) (1 + 2 * ((scales[ib / 2] >> (4 * (ib & 1))) & 0xF)));
        for (int k = 0; k < 8; ++k) {
            const uint32_t g = g_grid_prep[qs[8 * ib + k] | (((qh[ib] >> k) & 1) << 8)];
            const int l = k >> 1, half = k & 1;
            for (int j = 0; j < 4; ++j) {
                const float sg = (signs[4 * ib + l] >> (4 * half + j)) & 1 ? -1.f : 1.f;
                o[32 * ib + 8 * l + 4 * half + j] = __fmul_rn(__fmul_rn(db, (float) ((g >> (8 * j)) & 255u)), sg);
            }
        }
    }
}

// Fixture quantiser, the CUDA twin of the CPU checker's: d = f16(amax / 465); per 32-weight sub-block the scale
// candidates s0 - 1, s0, s0 + 1 around amax_sb / (15 d); per 4-weight group the nearest codebook row in 1/16-unit
// fixed point (ties: lower index); the candidate with the least total error (ties: the smallest s).  One thread per
// 4-weight group, 256 threads = 4 blocks of 256 weights.
__global__ void __launch_bounds__(256) k_quantize(const float* __restrict__ w, uint8_t* __restrict__ out, size_t nblocks) {
    __shared__ uint32_t grid[512];
    __shared__ uint8_t blk[4][112];
    const int tid = threadIdx.x;
    for (int i = tid; i < 512; i += 256) grid[i] = g_grid_prep[i];
    for (int i = tid; i < 4 * 112; i += 256) (&blk[0][0])[i] = 0;
    __syncthreads();
    const int lb = tid >> 6, grp = tid & 63, ib = grp >> 3, gi = grp & 7;   // block in CTA, group, sub-block, group in it
    const size_t b = (size_t) blockIdx.x * 4 + lb;
    const bool live = b < nblocks;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
        const float4 t = *reinterpret_cast<const float4*>(w + b * 256 + grp * 4);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    float am = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    // sub-block maximum over its 8 threads, block maximum over its 64 (two warps)
    float am_sb = am;
    for (int o = 4; o; o >>= 1) am_sb = fmaxf(am_sb, __shfl_xor_sync(0xffffffffu, am_sb, o));
    __shared__ float wmax_[8];
    float am_w = am_sb;
    for (int o = 16; o >= 8; o >>= 1) am_w = fmaxf(am_w, __shfl_xor_sync(0xffffffffu, am_w, o));
    if ((tid & 31) == 0) wmax_[tid >> 5] = am_w;
    __syncthreads();
    const float amax = fmaxf(wmax_[2 * lb], wmax_[2 * lb + 1]);
    const __half dh = __float2half_rn(__fdiv_rn(amax, 465.0f));
    const float d = __half2float(dh);
    if (d > 0.f) {
        const float t0 = __fmul_rn(__fsub_rn(__fdiv_rn(am_sb, __fmul_rn(15.0f, d)), 1.0f), 0.5f);
        int s0 = __float2int_rn(t0);
        s0 = max(0, min(15, s0));
        long long best_err = -1;
        int best_s = 0, best_idx = 0;
        for (int c = -1; c <= 1; ++c) {
            const int s = s0 + c;
            const bool valid = s >= 0 && s <= 15;   // every lane runs the search: the shuffles below are warp-wide
            const float sc = __fmul_rn(d, (float) (1 + 2 * s));
            int mi[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int q = __float2int_rn(__fmul_rn(__fdiv_rn(fabsf(v[j]), sc), 16.0f));
                mi[j] = min(q, 272);
            }
            int be = 0x7fffffff, bi = 0;
            for (int e = 0; e < 512; ++e) {
                const uint32_t g = grid[e];
                int ee = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int df = mi[j] - 16 * (int) ((g >> (8 * j)) & 255u);
                    ee += df * df;
                }
                if (ee < be) { be = ee; bi = e; }
            }
            long long err = be;
            for (int o = 4; o; o >>= 1) err += __shfl_xor_sync(0xffffffffu, err, o);
            err *= (long long) (1 + 2 * s) * (1 + 2 * s);
            if (valid && (best_err < 0 || err < best_err)) { best_err = err; best_s = s; best_idx = bi; }
        }
        // pack: this thread's index is number gi of sub-block ib; its 4 signs are bits 4 (gi & 1) .. of signs[4 ib + gi / 2]
        uint8_t* p = blk[lb];
        p[2 + 8 * ib + gi] = (uint8_t) (best_idx & 255);
        unsigned sgn = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) sgn |= (v[j] < 0.f ? 1u : 0u) << j;
        // qh bit, sign nibble and scale nibble are sub-byte fields shared by neighbouring threads: gather them with shuffles
        const unsigned hb = (unsigned) (best_idx >> 8) & 1u;
        unsigned qhb = hb << gi;
        for (int o = 4; o; o >>= 1) qhb |= __shfl_xor_sync(0xffffffffu, qhb, o);
        unsigned sb_ = sgn << (4 * (gi & 1));
        sb_ |= __shfl_xor_sync(0xffffffffu, sb_, 1);
        if (gi == 0) p[66 + ib] = (uint8_t) qhb;
        if ((gi & 1) == 0) p[74 + 4 * ib + (gi >> 1)] = (uint8_t) sb_;
        unsigned scn = (unsigned) best_s << (4 * (ib & 1));
        scn |= __shfl_xor_sync(0xffffffffu, scn, 8);   // sub-block ib ^ 1 sits 8 lanes away
        if (gi == 0 && (ib & 1) == 0) p[106 + ib / 2] = (uint8_t) scn;
        if (grp == 0) {
            const unsigned short hbits = __half_as_ushort(dh);
            p[0] = (uint8_t) (hbits & 255);
            p[1] = (uint8_t) (hbits >> 8);
        }
    }
    __syncthreads();
    if (live)
        for (int i = grp; i < IQ3S_BLOCK_BYTES; i += 64) out[b * IQ3S_BLOCK_BYTES + i] = blk[lb][i];
}

__global__ void k_fill_normal(float* __restrict__ out, size_t n, float sigma, uint32_t k0, uint32_t k1, uint32_t stream_id) {
    const size_t c = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (c * 4 >= n) return;
    uint32_t r[4];
    philox4x32_10((uint32_t) c, (uint32_t) (c >> 32), stream_id, 0u, k0, k1, r);
    float z[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const float u1 = ((float) (r[2 * h] >> 8) + 0.5f) * (1.0f / 16777216.0f);
        const float u2 = ((float) (r[2 * h + 1] >> 8) + 0.5f) * (1.0f / 16777216.0f);
        const float rad = sqrtf(-2.0f * logf(u1));
        float sn, cs;
        sincosf(6.283185307179586f * u2, &sn, &cs);
        z[2 * h] = rad * cs;
        z[2 * h + 1] = rad * sn;
    }
    for (int i = 0; i < 4 && c * 4 + i < n; ++i) out[c * 4 + i] = sigma * z[i];
}

}  // namespace fnxb

using namespace fnxb;

extern "C" size_t fnx_iq3s_bytes(size_t rows, size_t cols) { return iq3s_bytes(rows, cols); }

static int check_shape(const char* who, size_t rows, size_t cols) {
    if (rows == 0 || rows % 16 || cols == 0 || cols % 256) return fail(FNX_E_ARG, "%s: %zu x %zu is not a whole number of 16 x 256 tiles", who, rows, cols);
    return FNX_OK;
}

extern "C" int fnx_iq3s_retile(const void* ggml_blocks, void* tiles, size_t rows, size_t cols, fnx_stream st) {
    if (int rc = check_shape("fnx_iq3s_retile", rows, cols)) return rc;
    FNX_REQUIRE(ggml_blocks && tiles, "fnx_iq3s_retile: null pointer");
    const size_t n = rows * (cols / 256);
    k_retile<<<(unsigned) ((n + 127) / 128), 128, 0, as_stream(st)>>>((const uint8_t*) ggml_blocks, (uint8_t*) tiles, rows, (int) (cols / 256), 0);
    FNX_LAUNCH_OK("fnx_iq3s_retile");
    return FNX_OK;
}

extern "C" int fnx_iq3s_untile(const void* tiles, void* ggml_blocks, size_t rows, size_t cols, fnx_stream st) {
    if (int rc = check_shape("fnx_iq3s_untile", rows, cols)) return rc;
    FNX_REQUIRE(ggml_blocks && tiles, "fnx_iq3s_untile: null pointer");
    const size_t n = rows * (cols / 256);
    k_retile<<<(unsigned) ((n + 127) / 128), 128, 0, as_stream(st)>>>((const uint8_t*) ggml_blocks, (uint8_t*) tiles, rows, (int) (cols / 256), 1);
    FNX_LAUNCH_OK("fnx_iq3s_untile");
    return FNX_OK;
}

extern "C" int fnx_iq3s_dequant_tiles(const void* tiles, float* out, size_t rows, size_t cols, fnx_stream st) {
    if (int rc = check_shape("fnx_iq3s_dequant_tiles", rows, cols)) return rc;
    FNX_REQUIRE(tiles && out, "fnx_iq3s_dequant_tiles: null pointer");
    const size_t n = rows * (cols / 256);
    k_dequant_tiles<<<(unsigned) ((n + 127) / 128), 128, 0, as_stream(st)>>>((const uint8_t*) tiles, out, rows, (int) (cols / 256));
    FNX_LAUNCH_OK("fnx_iq3s_dequant_tiles");
    return FNX_OK;
}

extern "C" int fnx_iq3s_quantize(const float* w, void* ggml_blocks, size_t n, fnx_stream st) {
    FNX_REQUIRE(w && ggml_blocks && n && n % 256 == 0, "fnx_iq3s_quantize: %zu values is not a whole number of 256-weight blocks", n);
    const size_t nb = n / 256;
    k_quantize<<<(unsigned) ((nb + 3) / 4), 256, 0, as_stream(st)>>>(w, (uint8_t*) ggml_blocks, nb);
    FNX_LAUNCH_OK("fnx_iq3s_quantize");
    return FNX_OK;
}

extern "C" int fnx_fill_normal(float* out, size_t n, float sigma, uint64_t seed, uint32_t stream_id, fnx_stream st) {
    FNX_REQUIRE(out && n, "fnx_fill_normal: nothing to fill");
    const size_t nc = (n + 3) / 4;
    k_fill_normal<<<(unsigned) ((nc + 255) / 256), 256, 0, as_stream(st)>>>(out, n, sigma, (uint32_t) seed, (uint32_t) (seed >> 32), stream_id);
    FNX_LAUNCH_OK("fnx_fill_normal");
    return FNX_OK;
}
