// Interface of the tensor-core decode attention kernel (attention_decode_mma.cu) towards
// the dispatcher in attention_generic.cu.
#pragma once

#include "common.cuh"

namespace ems {

struct DecodeParams {
    const bf16* q;      // [N, q_stride], first nh*D columns
    bf16* out;          // [N, nh*D]
    const bf16* kc;     // [pages, nkv, page_size, D]
    const bf16* vc;
    const int* bt;      // [B, bt_stride]
    const int* cu_q;    // [B+1] packed token index of each row (rows have one token)
    const int* starts;  // [B] keys cached before this step; the query stands at that position
    float* part_o;      // [N*nh, splits, D]
    float* part_ml;     // [N*nh, splits, 2]  (max in natural-log units, sum)
    long long q_stride;
    int bt_stride, page_size, nh, nkv, G, window, splits;
    float scale_log2;   // log2(e) / sqrt(D)
    // The fused decode form (attention_decode_mma.cu): `q` is the raw qkv row [q | k | v]; the
    // kernel rotates q (and k) itself with `rope_table` [positions, rot / 2, (cos, sin)] and, with
    // write_kv, puts the row's new key and value into the cache (and into its own tile of them).
    const float* rope_table = nullptr;
    int rot = 0;        // 0 (no rotation) or D
    int fused = 0;
    int write_kv = 0;
    // Beyond the plain causal form, in the kernels that say they take it (all optional):
    int chunk = 0;                  // > 0: the query at p sees only keys j with j / chunk == p / chunk
    const float* sinks = nullptr;   // [nh]: exp(sinks[h]) joins the softmax's denominator
    const bf16* gate = nullptr;     // [N, gate_stride]: head h's output times sigmoid(gate[n, h])
    long long gate_stride = 0;
    int keep = 0;                   // > 0: keys j < keep stay visible beside the window
    const float* out_table = nullptr;  // [positions, D / 2, (cos, sin)]: the result is turned back by the query's position
    int out_pairing = 0;            // 0: pair (i, i + D / 2); 1: pair (2 i, 2 i + 1)
    const int* positions = nullptr; // [N] position of each token of the step
    float softcap = 0.f;            // > 0: a score s (already scaled) becomes softcap * tanh(s / softcap)
    float scale = 0.f;              // the plain score scale (scale_log2 / log2(e)), read with softcap
};

// The key tiles that a block walks when the first `keep` keys stay visible beside the window: `nhead`
// tiles from position 0 (those that lie wholly before the window's first tile), then the tiles from kt0.
__host__ __device__ __forceinline__ int tile_start(int t, int nhead, int kt0, int bk) {
    return t < nhead ? t * bk : kt0 + (t - nhead) * bk;
}

// The first key that the query at position p may see.
__host__ __device__ __forceinline__ int first_visible(int p, int window, int chunk) {
    int lo = window > 0 ? (p - window + 1 > 0 ? p - window + 1 : 0) : 0;
    if (chunk > 0 && (p / chunk) * chunk > lo) lo = (p / chunk) * chunk;
    return lo;
}

bool decode_mma_supported(int dtype, int D, int G, long long q_stride, const void* q, const void* kc,
                          const void* vc);
int run_decode_mma(const DecodeParams& p, int B, int D, cudaStream_t stream);
bool decode_fused_supported(int D, int G, int rot, long long q_stride, const void* q, const void* kc,
                            const void* vc);

// The tensor-core kernel for prompt portions and mixed rows (attention_prefill_mma.cu);
// it uses the same parameter block (no split of the keys: part_o / part_ml unused).
bool prefill_mma_supported(int dtype, int D, long long q_stride, const void* q, const void* out,
                           const void* kc, const void* vc);
int run_prefill_mma(const DecodeParams& p, int B, int D, int max_q_len, cudaStream_t stream);
// The same kernel with a chunk mask, sinks, a gate per head, kept first keys and a result that is turned
// back (DecodeParams::chunk, sinks, gate, keep, out_table); the
// softmax weights enter the second product as two bfloat16 terms (value and remainder), so that they
// carry 16 bits of mantissa instead of 8.
int run_prefill_mma_masked(const DecodeParams& p, int B, int D, int max_q_len, cudaStream_t stream);

// The tcgen05 kernel for prompt portions (attention_prefill_tc05.cu): long prompts at head
// sizes 64 and 128 with pages of a multiple of 16 keys; same parameter block.
bool prefill_tc05_supported(int dtype, int D, int page_size, long long q_stride, const void* q, const void* out,
                            const void* kc, const void* vc);
int run_prefill_tc05(const DecodeParams& p, int B, int D, int max_q_len, cudaStream_t stream);

}  // namespace ems
