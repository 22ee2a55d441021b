// The verify window as one persistent kernel (window.cu): parameter blocks shared with the host scheduler (engine.cu).
#pragma once

#include <cuda_fp16.h>

#include "fnx_common.cuh"

namespace fnxb {

constexpr int WIN_THREADS = 512;
constexpr int WIN_MAX_ROWS = 8;      // rows of a window the kernel takes (two groups of four rows per tile product)
constexpr int WIN_SYNC_WORDS = 8;    // [0] the grid barrier's arrival counter
constexpr int WIN_PROF_WORDS = 4096;
constexpr int WIN_MAX_LAYERS = 64;

struct WinLayer {
    int attn, in_rows;
    const float *norm1, *norm2;
    const uint8_t *w_in, *w_out;
    const float *qn, *kn;
    __half *kc, *vc;
    const float *convw, *dt, *a, *gnorm;
    float *S, *hist;
    const float* wr;
    const uint8_t *wgu, *wdn, *wsh_gu, *wsh_dn;
};

// Expert-parallel exchange of the window kernel (ranks > 1): every rank's landing planes [2 slots][ranks][rows][H] of
// fixed-point sums and arrival flags [2 slots][ranks][blocks], mapped into every rank (peer memory over NVLink).
struct WinPeers {
    unsigned long long* x[8];
    unsigned* flag[8];
};

// The whole parameter block is passed to the kernel BY VALUE (a __grid_constant__ parameter of ~10 KB): its fields are
// constant-bank operands, which cost no registers and which the compiler can re-read instead of spilling.
struct WinParams {
    int n_layer;
    int H, E, K, F, nq, nkv, hd, nrot, nk, nv, hs, V;
    int T, NS, proj_ld, tree;
    int e_lo, e_hi, e_base;          // this rank's experts [e_lo, e_hi); e_base = the first expert held at wgu / wdn
    int ep_rank, ep_size, maxr;
    float eps, rope_base;
    size_t gu_bytes, dn_bytes;
    const int *tok, *parent, *pos0, *cur;
    int* depth;
    const __half* embed;
    const uint8_t* head;
    const float* out_norm;
    int head_row0;                   // the head is applied to rows [head_row0, T) (the draft layer: the last row only)
    float *R, *proj, *mix, *logits, *rlogits, *topw, *hbuf;
    int* topi;
    fnx_job* jobs;
    int* njobs;
    float* att_acc;
    void* att_mz;
    float *gdn_o, *gdn_sq;
    unsigned long long* racc;        // [T][H] fixed-point sums of the expert block's addends
    unsigned* sync;
    unsigned long long* stats;
    unsigned* err;
    unsigned long long* prof;
    // the draft layer's input: R = fc_hid(rms(src)) + fc_emb(rms(emb(tok))) instead of the token embeddings
    int dbg;                         // tracing aid: 1 = the input projection and the router phases run twice (cold against warm)
    int mtp;
    const uint8_t *fc_hid, *fc_emb;
    const float *hnorm, *enorm;
    const float* src;
    float* emb;
    // expert parallel
    WinPeers peers;
    unsigned* xseq;                  // [0] exchanges so far (the slot's parity and the flags' value)
    WinLayer layers[WIN_MAX_LAYERS];
};

size_t win_smem_bytes();
// One window of T <= WIN_MAX_ROWS rows: embeddings (or the draft layer's input), every layer, the head.  Leaves the
// logits of rows [head_row0, T) and the final residual rows in place; capture-safe (a memset node and one cooperative launch).
int win_launch(const WinParams& params, unsigned* sync_words, cudaStream_t st);
// per device, before any capture: raises the kernel's shared-memory limit
int win_setup();

}  // namespace fnxb
