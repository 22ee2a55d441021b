// Parameter blocks of the persistent verify-step kernel (step.cu), shared with the engine that fills them.
#pragma once

#include <cuda_fp16.h>

#include <cstdint>

#include "../../include/fnx_b200.h"

namespace fnxb {

struct StepLayer {
    int attn;
    int in_rows;
    const float *norm1, *norm2;
    const uint8_t *w_in, *w_out;
    const float *qn, *kn;
    __half *kc, *vc;                 // this sequence's caches
    const float *convw, *dt, *a, *gnorm;
    float *S, *hist;                 // this sequence's state and conv-history rings
    const float* wr;
    const uint8_t *wgu, *wdn, *wsh_gu, *wsh_dn;
};

struct AttPartialS {
    float m, z;
};

struct StepParams {
    const StepLayer* layers;
    int n_layer;
    int H, E, K, F, nq, nkv, hd, nrot, nk, nv, hs, V;
    int T, NS, proj_ld, tree;
    float eps, rope_base;
    size_t gu_bytes, dn_bytes;
    // window inputs and scalars (device)
    const int *tok, *parent, *pos0, *cur;
    int* depth;
    const __half* embed;
    const uint8_t* head;
    const float* out_norm;
    // buffers
    float *R, *proj, *mix, *logits, *rlogits, *topw, *hbuf, *part;
    int* topi;
    fnx_job* jobs;
    int* njobs;
    float* att_acc;
    AttPartialS* att_mz;
    float *gdn_o, *gdn_sq;
    uint8_t* ximg;       // quantised activation image for the next matrix phase
    float* xnorm;        // f32 normalised rows for the router
    int* best_i;
    float* best_v;
    int* result;
    unsigned* sync;      // [0] grid barrier counter, [1..] last-block counters; zeroed before every launch
    unsigned long long* stats;
    unsigned* err;
    unsigned long long* prof;   // optional phase stamps of block 0
};

constexpr int STEP_SYNC_WORDS = 16;
constexpr int STEP_THREADS = 512;
size_t step_smem_bytes();
// enqueues the zeroing of the sync words and the cooperative launch; `dev_params` is a device copy of StepParams
int step_launch(const StepParams* dev_params, int T, unsigned* sync_words, cudaStream_t st);

}  // namespace fnxb
