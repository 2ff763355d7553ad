// Parameter block of the persistent decode-step kernel (decode_mega.cu).
#pragma once
#include <cuda.h>
#include "lc_kernels.h"
#include "lc_attn.cuh"

namespace lc {

enum MegaPhaseType { PH_GEMV = 0, PH_ATTN = 1, PH_ARGMAX = 2, PH_FINAL = 3, PH_EMBED = 4 };

struct MegaPhase {
    int type;        // MegaPhaseType
    int n, k;        // PH_GEMV: output rows, inputs
    int tm0, tm1;    // indices into MegaParams::tmaps (tm1 = -1 unless the phase is the gate/up pair)
    int epi;         // GemvEpilogue
    int layer;       // PH_ATTN: which KV pools
    int reserved;
    const float* x;
    float* out;
    const float* residual;
    const float* norm_w;
};

struct MegaParams {
    const CUtensorMap* tmaps;   // device array, 64-byte aligned entries
    const MegaPhase* phases;    // device array
    int n_phases;
    int max_units;              // largest k / 256 over the matrix phases
    AttnParams attn;            // pools are taken per layer from k_pools / v_pools
    void* const* k_pools;
    void* const* v_pools;
    const uint8_t* embed;       // token embedding table (raw blocks), rows of H elements
    uint32_t embed_typ;
    int64_t embed_rows;
    int64_t* tokens;            // [1] current token id; overwritten with the greedy pick
    float* hidden;              // [H] residual stream
    const float* logits;        // [V]
    int V;
    int64_t* next;              // [1]
    int32_t* tok_pos;           // [1] cache position, advanced at the end of the step
    int32_t* tok_rope;          // [1]
    int rope_absolute;
    int64_t* out_tokens;        // log of picks, indexed by *step_ctr (may be null)
    int32_t* step_ctr;
    long long* argmax_scratch;  // [grid]
    unsigned long long* bar;    // grid barrier arrival counter (never reset)
    int* error_flag;
    float eps;
    unsigned long long* trace;  // optional [n_phases][2] globaltimer stamps of CTA 0: phase entered (after the barrier), phase done
};

size_t decode_mega_smem_bytes(int max_units);
int32_t launch_decode_mega(const MegaParams& P, cudaStream_t s);
// split of the context that launch_attention would use for these sizes
void attention_plan(int n_tok, int n_heads, int max_ctx, int* chunk, int* n_splits);

}  // namespace lc
