// Kernels of layers whose two sub-layers read the same normed stream, of the delta-rule memory, and of a
// selective state space:
//
//  * ems_add_scaled_norm2: residual += sum_i scale_i * delta_i (up to three deltas, 32-bit sum), then
//    one root mean square of the new residual serves two norms with gains of their own (a block whose
//    mixer and feed-forward both read norm(x)); every part is optional;
//  * ems_stream_norm: the 32-bit stream itself is RMS-normed in place (a norm behind the embedding);
//  * ems_softcap: x <- cap * tanh(x / cap) on 32-bit values (logits);
//  * ems_delta_recurrence: a matrix memory per head written by the delta rule with a decay per key
//    channel, S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//    (Schlag, Irie, Schmidhuber, "Linear Transformers Are Secretly Fast Weight Programmers", with the
//    gate of Yang, Kautz, Hatamizadeh, "Gated Delta Networks: Improving Mamba2 with Delta Rule", taken
//    per channel);
//  * ems_ssm_gates: step size and decay of a selective state space with a scalar decay per head
//    (Dao, Gu, "Transformers are SSMs: Generalized Models and Efficient Algorithms Through Structured
//    State Space Duality"): dt = softplus(x + bias), a = exp(-exp(A_log) dt), b = dt;
//  * ems_gate_group_norm: what follows that state space's read: (o + D_h act(x)) * silu(z), then an
//    RMS norm in equal groups with a gain.
//
// States, decays, gates, unit norms and every product with a state are 32-bit; projections and
// convolution outputs arrive in the activation type and are widened once.  A request's tokens are
// walked in order by the same code in prompts, portions and single tokens.
#include "common.cuh"

namespace ems {

__device__ __forceinline__ float d_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float d_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float d_silu(float z) { return z / (1.f + expf(-z)); }

// ---------------------------------------------------------------------------------------
// residual += s0 d0 + s1 d1 + s2 d2;  r = rsqrt(mean(residual^2) + eps);  out1 = residual r g1;  out2 = residual r g2
// (gains are read as stored plus `gain_offset`); without outputs the sum alone.

template <typename T>
__global__ void add_scaled_norm2_kernel(const T* __restrict__ d0, const T* __restrict__ d1, const T* __restrict__ d2,
                                        float s0, float s1, float s2, float* __restrict__ residual,
                                        const void* __restrict__ g1, const void* __restrict__ g2, int g_dtype,
                                        float gain_offset, float eps, T* __restrict__ out1, T* __restrict__ out2,
                                        int C) {
    __shared__ float red[33];
    const size_t base = (size_t)blockIdx.x * C;
    float ss = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float x = residual[base + c];
        if (d0 || d1 || d2) {
            if (d0) x = fmaf(s0, to_f32<T>(d0[base + c]), x);
            if (d1) x = fmaf(s1, to_f32<T>(d1[base + c]), x);
            if (d2) x = fmaf(s2, to_f32<T>(d2[base + c]), x);
            residual[base + c] = x;
        }
        ss = fmaf(x, x, ss);
    }
    if (!out1 && !out2) return;
    const float r = rsqrtf(block_sum(ss, red) / C + eps);
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float x = residual[base + c] * r;  // (this thread wrote it)
        if (out1) out1[base + c] = from_f32<T>(x * (load_any(g1, g_dtype, c) + gain_offset));
        if (out2) out2[base + c] = from_f32<T>(x * (load_any(g2, g_dtype, c) + gain_offset));
    }
}

__global__ void stream_norm_kernel(float* __restrict__ residual, const void* __restrict__ gain, int g_dtype,
                                   float gain_offset, float eps, int C) {
    __shared__ float red[33];
    const size_t base = (size_t)blockIdx.x * C;
    float ss = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) ss = fmaf(residual[base + c], residual[base + c], ss);
    const float r = rsqrtf(block_sum(ss, red) / C + eps);
    for (int c = threadIdx.x; c < C; c += blockDim.x)
        residual[base + c] = residual[base + c] * r * (load_any(gain, g_dtype, c) + gain_offset);
}

__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] / cap);
}

// ---------------------------------------------------------------------------------------
// the delta-rule memory
//
// Two kernels.  ems::delta_prep_kernel computes, once per token, what the recurrence reads: q and k of
// every q / k head (activation, unit norm, the query's scale), k . q, the decay of every head and key
// channel, beta, and the activation of v; all 32-bit, in a work buffer [N, 2 HK D + H D + H V + HK + H]
// (q | k | g | v | k.q | beta).
// ems::delta_recurrence_kernel then walks the tokens: as in the matrix memory of recurrent.cu, a block
// owns a group of columns of one head's S ([D, V]) for one request; a column is shared by SL
// lanes, lane s holding rows i * 4 SL + 4 s + e of the column in registers, and a lane holds its rows of
// two columns, so that the rows of q, k and g it reads from shared memory serve both.  Tiles of 32 tokens of q, k
// and g are copied into shared memory with cp.async, the next tile while this one is computed.  A
// column's update needs S^T k before it can write, so that dot product closes with shuffles for every
// token; the read o = S^T q = (g S)^T q + u (k.q) is linear in what a lane holds, so the lanes' shares
// are summed once per tile.

constexpr int DR_WARPS = 8;
constexpr int DR_TT = 32;
constexpr int DR_CPL = 2;   // columns of S per lane: what a lane reads of q, k and g serves both

struct DeltaParams {
    const void* q; const void* k; const void* v;   // [N, ld*] views; q/k head j begins at column j * D, v head h at h * V
    long long ldq, ldk, ldv;
    const void* beta;          // [N, ldb] activation type: beta = sigmoid(beta[t, h])
    long long ldb;
    const float* g_raw;        // [N, H * D] float: decay pre-activations without their bias
    const void* g_bias;        // [H * D]
    const void* a_log;         // [H]: g = exp(-exp(a_log[h]) * softplus(g_raw + g_bias))
    int p_dtype;               // element type of g_bias and a_log
    float* work;               // [N, work_ld]: q [HK * D] | k [HK * D] | g [H * D] | v [H * V] | k.q [HK] | beta [H]
    int work_ld;
    float* state;              // [slots, H, D * V]
    const int* slots; const int* cu_q;
    float* out;                // [N, H * V] float
    int H, HK, D, V, act, unit, vec_ok;
    float q_scale, unit_eps;
};

__device__ __forceinline__ float dr_in(float z, int act) { return act ? d_silu(z) : z; }

// one block per token; a warp per head at a time
template <typename T>
__global__ void delta_prep_kernel(const DeltaParams p) {
    const int tok = blockIdx.x, D = p.D;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    float* w = p.work + (size_t)tok * p.work_ld;
    float* wq = w;
    float* wk = wq + (size_t)p.HK * D;
    float* wg = wk + (size_t)p.HK * D;
    float* wv = wg + (size_t)p.H * D;
    float* wkq = wv + (size_t)p.H * p.V;
    float* wb = wkq + p.HK;
    {
        const T* vg = reinterpret_cast<const T*>(p.v) + (size_t)tok * p.ldv;
        for (int c = threadIdx.x; c < p.H * p.V; c += blockDim.x) wv[c] = dr_in(to_f32<T>(vg[c]), p.act);
    }
    for (int j = warp; j < p.HK + p.H; j += nwarps) {
        if (j < p.HK) {
            const T* qg = reinterpret_cast<const T*>(p.q) + (size_t)tok * p.ldq + (size_t)j * D;
            const T* kg = reinterpret_cast<const T*>(p.k) + (size_t)tok * p.ldk + (size_t)j * D;
            float sq = 0.f, sk = 0.f, qk = 0.f;
            for (int d = lane; d < D; d += 32) {
                const float a = dr_in(to_f32<T>(qg[d]), p.act), b = dr_in(to_f32<T>(kg[d]), p.act);
                sq = fmaf(a, a, sq);
                sk = fmaf(b, b, sk);
                qk = fmaf(a, b, qk);
            }
            sq = warp_sum(sq);
            sk = warp_sum(sk);
            qk = warp_sum(qk);
            const float rq = (p.unit ? rsqrtf(sq + p.unit_eps) : 1.f) * p.q_scale;
            const float rk = p.unit ? rsqrtf(sk + p.unit_eps) : 1.f;
            for (int d = lane; d < D; d += 32) {
                wq[(size_t)j * D + d] = dr_in(to_f32<T>(qg[d]), p.act) * rq;
                wk[(size_t)j * D + d] = dr_in(to_f32<T>(kg[d]), p.act) * rk;
            }
            if (lane == 0) wkq[j] = qk * rq * rk;
        } else {
            const int h = j - p.HK;
            const float neg_a = -expf(load_any(p.a_log, p.p_dtype, h));
            for (int d = lane; d < D; d += 32) {
                const size_t ch = (size_t)h * D + d;
                wg[ch] = expf(neg_a * d_softplus(p.g_raw[(size_t)tok * ((size_t)p.H * D) + ch] + load_any(p.g_bias, p.p_dtype, ch)));
            }
            if (lane == 0) wb[h] = d_sigmoid(to_f32<T>(reinterpret_cast<const T*>(p.beta)[(size_t)tok * p.ldb + h]));
        }
    }
}

__device__ __forceinline__ void dr_cp4(float* dst, const float* src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 4 : 0;   // (0: the word is filled with zeros)
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}

__device__ __forceinline__ void dr_cp16(float* dst, const float* src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;   // (0: the 16 bytes are filled with zeros)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}

template <typename T, int DPT, int SL>
__global__ void __launch_bounds__(DR_WARPS * 32) delta_recurrence_kernel(const DeltaParams p) {
    constexpr int TT = DR_TT;
    constexpr int THREADS = DR_WARPS * 32;
    constexpr int DP = SL * DPT;
    constexpr int WCOLS = 32 / SL;
    constexpr int GCOLS = DR_WARPS * WCOLS;                   // columns of one pass over the warps
    constexpr int COLS = GCOLS * DR_CPL;                      // columns of a block
    constexpr int STAGE = 3 * TT * DP + TT * COLS + 2 * TT;   // floats of one stage
    extern __shared__ __align__(16) float smem[];
    const int D = p.D, V = p.V;
    const int row = blockIdx.z, head = blockIdx.y;
    const int kh = head / (p.H / p.HK);
    const int q0 = p.cu_q[row], qlen = p.cu_q[row + 1] - q0;
    if (qlen <= 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slice = lane & (SL - 1), colw = lane / SL;
    const int lcol = warp * WCOLS + colw;                      // this lane's first column inside the block
    float* st = p.state + ((size_t)p.slots[row] * p.H + head) * ((size_t)D * V);
    float S[DR_CPL][DPT];
#pragma unroll
    for (int c = 0; c < DR_CPL; ++c) {
        const int col = blockIdx.x * COLS + lcol + c * GCOLS;
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = (i / 4) * (4 * SL) + 4 * slice + (i & 3);
            S[c][i] = (col < V && d < D) ? st[(size_t)d * V + col] : 0.f;
        }
    }
    const size_t off_q = (size_t)kh * D, off_k = (size_t)p.HK * D + (size_t)kh * D;
    const size_t off_g = 2 * (size_t)p.HK * D + (size_t)head * D;
    const size_t off_v = 2 * (size_t)p.HK * D + (size_t)p.H * D + (size_t)head * V + (size_t)blockIdx.x * COLS;
    const size_t off_kq = 2 * (size_t)p.HK * D + (size_t)p.H * D + (size_t)p.H * V + kh;
    const size_t off_b = 2 * (size_t)p.HK * D + (size_t)p.H * D + (size_t)p.H * V + p.HK + head;

    // Stage the tile that begins at token t0: q, k, g rows (zeros past D; tokens past the end hold q = k = 0,
    // g = 1, beta = 0: nothing changes), v of this block's columns, k.q and beta.
    auto stage = [&](int t0, float* buf) {
        const int cnt = min(TT, qlen - t0);
        float* qs = buf;
        float* ks = qs + TT * DP;
        float* gs = ks + TT * DP;
        float* vs = gs + TT * DP;
        float* bs = vs + TT * COLS;
        float* kqs = bs + TT;
        if (p.vec_ok) {
            for (int idx = threadIdx.x; idx < TT * (DP / 4); idx += THREADS) {
                const int t = idx / (DP / 4), d = (idx % (DP / 4)) * 4;
                const bool ok = t < cnt && d < D;
                const float* w = p.work + (size_t)(q0 + t0 + (ok ? t : 0)) * p.work_ld + (ok ? d : 0);
                dr_cp16(qs + t * DP + d, w + off_q, ok);
                dr_cp16(ks + t * DP + d, w + off_k, ok);
                if (ok) dr_cp16(gs + t * DP + d, w + off_g, true);
                else *reinterpret_cast<float4*>(gs + t * DP + d) = make_float4(1.f, 1.f, 1.f, 1.f);
            }
        } else {
            for (int idx = threadIdx.x; idx < TT * DP; idx += THREADS) {
                const int t = idx / DP, d = idx % DP;
                const bool ok = t < cnt && d < D;
                const float* w = p.work + (size_t)(q0 + t0 + (ok ? t : 0)) * p.work_ld + (ok ? d : 0);
                qs[idx] = ok ? w[off_q] : 0.f;
                ks[idx] = ok ? w[off_k] : 0.f;
                gs[idx] = ok ? w[off_g] : 1.f;
            }
        }
        if (p.vec_ok) {   // (V is a multiple of 4 then: a group of four columns lies inside the head or outside)
            for (int idx = threadIdx.x; idx < TT * (COLS / 4); idx += THREADS) {
                const int t = idx / (COLS / 4), c = (idx % (COLS / 4)) * 4;
                const bool ok = t < cnt && (int)(blockIdx.x * COLS) + c < V;
                const float* w = p.work + (size_t)(q0 + t0 + (ok ? t : 0)) * p.work_ld + off_v + (ok ? c : 0);
                dr_cp16(vs + t * COLS + c, ok ? w : p.work, ok);
            }
            if ((int)threadIdx.x < 2 * TT) {
                const int t = threadIdx.x % TT;
                const bool ok = t < cnt;
                const float* w = p.work + (size_t)(q0 + t0 + (ok ? t : 0)) * p.work_ld;
                dr_cp4((int)threadIdx.x < TT ? bs + t : kqs + t, w + ((int)threadIdx.x < TT ? off_b : off_kq), ok);
            }
        } else {
            for (int idx = threadIdx.x; idx < TT * COLS; idx += THREADS) {
                const int t = idx / COLS, c = idx % COLS;
                const bool ok = t < cnt && (int)(blockIdx.x * COLS) + c < V;
                vs[idx] = ok ? p.work[(size_t)(q0 + t0 + t) * p.work_ld + off_v + c] : 0.f;
            }
            if ((int)threadIdx.x < TT) {
                const int t = threadIdx.x;
                const float* w = p.work + (size_t)(q0 + t0 + (t < cnt ? t : 0)) * p.work_ld;
                bs[t] = t < cnt ? w[off_b] : 0.f;
                kqs[t] = t < cnt ? w[off_kq] : 0.f;
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

    stage(0, smem);
    int cur = 0;
    for (int t0 = 0; t0 < qlen; t0 += TT, cur ^= 1) {
        const int cnt = min(TT, qlen - t0);
        if (t0 + TT < qlen) {
            stage(t0 + TT, smem + (cur ^ 1) * STAGE);   // in flight while this tile is computed
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        const float* qs = smem + cur * STAGE;
        const float* ks = qs + TT * DP;
        const float* gs = ks + TT * DP;
        const float* vs = gs + TT * DP;
        const float* bs = vs + TT * COLS;
        const float* kqs = bs + TT;
        // A lane reads its rows of q, k and g once per token and uses them for each of its DR_CPL columns.
        float acc[DR_CPL][TT];
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            const float4* k4 = reinterpret_cast<const float4*>(ks + t * DP) + slice;
            const float4* q4 = reinterpret_cast<const float4*>(qs + t * DP) + slice;
            const float4* g4 = reinterpret_cast<const float4*>(gs + t * DP) + slice;
            float dk[DR_CPL], dq[DR_CPL], dk1[DR_CPL], dq1[DR_CPL];   // (two partial sums each: shorter chains)
#pragma unroll
            for (int c = 0; c < DR_CPL; ++c) dk[c] = dq[c] = dk1[c] = dq1[c] = 0.f;
            float4 kk[DPT / 4];
#pragma unroll
            for (int i = 0; i < DPT / 4; ++i) {
                const float4 qq = q4[i * SL], gg = g4[i * SL];
                kk[i] = k4[i * SL];
#pragma unroll
                for (int c = 0; c < DR_CPL; ++c) {
                    S[c][4 * i + 0] *= gg.x;
                    S[c][4 * i + 1] *= gg.y;
                    S[c][4 * i + 2] *= gg.z;
                    S[c][4 * i + 3] *= gg.w;
                    dk[c] = fmaf(S[c][4 * i + 0], kk[i].x, dk[c]);
                    dq[c] = fmaf(S[c][4 * i + 0], qq.x, dq[c]);
                    dk1[c] = fmaf(S[c][4 * i + 1], kk[i].y, dk1[c]);
                    dq1[c] = fmaf(S[c][4 * i + 1], qq.y, dq1[c]);
                    dk[c] = fmaf(S[c][4 * i + 2], kk[i].z, dk[c]);
                    dq[c] = fmaf(S[c][4 * i + 2], qq.z, dq[c]);
                    dk1[c] = fmaf(S[c][4 * i + 3], kk[i].w, dk1[c]);
                    dq1[c] = fmaf(S[c][4 * i + 3], qq.w, dq1[c]);
                }
            }
#pragma unroll
            for (int c = 0; c < DR_CPL; ++c) {
                dk[c] += dk1[c];
                dq[c] += dq1[c];
            }
#pragma unroll
            for (int off = SL / 2; off >= 1; off >>= 1)
#pragma unroll
                for (int c = 0; c < DR_CPL; ++c) dk[c] += __shfl_xor_sync(0xffffffffu, dk[c], off);
            const float beta = bs[t], kq = kqs[t];
#pragma unroll
            for (int c = 0; c < DR_CPL; ++c) {
                const float u = beta * (vs[t * COLS + lcol + c * GCOLS] - dk[c]);
#pragma unroll
                for (int i = 0; i < DPT / 4; ++i) {
                    S[c][4 * i + 0] = fmaf(kk[i].x, u, S[c][4 * i + 0]);
                    S[c][4 * i + 1] = fmaf(kk[i].y, u, S[c][4 * i + 1]);
                    S[c][4 * i + 2] = fmaf(kk[i].z, u, S[c][4 * i + 2]);
                    S[c][4 * i + 3] = fmaf(kk[i].w, u, S[c][4 * i + 3]);
                }
                acc[c][t] = dq[c] + (slice == 0 ? u * kq : 0.f);
            }
        }
        // the lanes' shares of the reads, summed once per tile (a lane hands one half of what it holds to
        // its partner and adds the partner's other half)
#pragma unroll
        for (int c = 0; c < DR_CPL; ++c) {
#pragma unroll
            for (int off = SL / 2, n = TT; off >= 1; off >>= 1, n >>= 1) {
                const bool upper = (lane & off) != 0;
#pragma unroll
                for (int j = 0; j < n / 2; ++j) {
                    const float send = upper ? acc[c][j] : acc[c][j + n / 2];
                    const float keep = upper ? acc[c][j + n / 2] : acc[c][j];
                    acc[c][j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
            const int col = blockIdx.x * COLS + lcol + c * GCOLS;
            if (col < V) {
#pragma unroll
                for (int j = 0; j < TT / SL; ++j) {
                    const int t = slice * (TT / SL) + j;
                    if (t < cnt) p.out[(size_t)(q0 + t0 + t) * ((size_t)p.H * V) + (size_t)head * V + col] = acc[c][j];
                }
            }
        }
        __syncthreads();  // this tile is consumed before the stage after next overwrites it
    }
#pragma unroll
    for (int c = 0; c < DR_CPL; ++c) {
        const int col = blockIdx.x * COLS + lcol + c * GCOLS;
        if (col >= V) continue;
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = (i / 4) * (4 * SL) + 4 * slice + (i & 3);
            if (d < D) st[(size_t)d * V + col] = S[c][i];
        }
    }
}

// A step in which every request brings one token: a thread owns a column of S and walks its rows twice
// (S^T k of the decayed state, then the write and the read), so that the lanes of a warp touch
// consecutive floats of every row.
template <typename T>
__global__ void __launch_bounds__(128) delta_step_kernel(const DeltaParams p) {
    __shared__ float qs[256], ks[256], gs[256];
    const int D = p.D, V = p.V;
    const int tok = blockIdx.z, head = blockIdx.y;   // (row r brings token r)
    const int kh = head / (p.H / p.HK);
    const float* w = p.work + (size_t)tok * p.work_ld;
    const float* wq = w + (size_t)kh * D;
    const float* wk = w + (size_t)p.HK * D + (size_t)kh * D;
    const float* wg = w + 2 * (size_t)p.HK * D + (size_t)head * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        qs[d] = wq[d];
        ks[d] = wk[d];
        gs[d] = wg[d];
    }
    __syncthreads();
    const int col = blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= V) return;
    const float beta = w[2 * (size_t)p.HK * D + (size_t)p.H * D + (size_t)p.H * V + p.HK + head];
    const float vj = w[2 * (size_t)p.HK * D + (size_t)p.H * D + (size_t)head * V + col];
    float* sp = p.state + ((size_t)p.slots[tok] * p.H + head) * ((size_t)D * V) + col;
    float dk0 = 0.f, dk1 = 0.f;
    int d = 0;
    for (; d + 1 < D; d += 2) {
        dk0 = fmaf(gs[d] * sp[(size_t)d * V], ks[d], dk0);
        dk1 = fmaf(gs[d + 1] * sp[(size_t)(d + 1) * V], ks[d + 1], dk1);
    }
    if (d < D) dk0 = fmaf(gs[d] * sp[(size_t)d * V], ks[d], dk0);
    const float u = beta * (vj - (dk0 + dk1));
    float o0 = 0.f, o1 = 0.f;
    for (d = 0; d + 1 < D; d += 2) {
        const float s0 = fmaf(ks[d], u, gs[d] * sp[(size_t)d * V]);
        const float s1 = fmaf(ks[d + 1], u, gs[d + 1] * sp[(size_t)(d + 1) * V]);
        sp[(size_t)d * V] = s0;
        sp[(size_t)(d + 1) * V] = s1;
        o0 = fmaf(s0, qs[d], o0);
        o1 = fmaf(s1, qs[d + 1], o1);
    }
    if (d < D) {
        const float s0 = fmaf(ks[d], u, gs[d] * sp[(size_t)d * V]);
        sp[(size_t)d * V] = s0;
        o0 = fmaf(s0, qs[d], o0);
    }
    p.out[(size_t)tok * ((size_t)p.H * V) + (size_t)head * V + col] = o0 + o1;
}

template <typename T, int DPT, int SL>
static int launch_delta_as(const DeltaParams& p, int rows, cudaStream_t stream) {
    constexpr int COLS = DR_WARPS * (32 / SL) * DR_CPL;
    const dim3 grid((p.V + COLS - 1) / COLS, p.H, rows);
    const size_t smem = sizeof(float) * 2 * ((size_t)DR_TT * (3 * SL * DPT + COLS) + 2 * DR_TT);
    auto kernel = delta_recurrence_kernel<T, DPT, SL>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return EMS_ERR_LAUNCH;
    kernel<<<grid, DR_WARPS * 32, smem, stream>>>(p);
    return launch_status();
}

template <typename T>
static int launch_delta(DeltaParams& p, int rows, int N, cudaStream_t stream) {
    const int units = p.HK + p.H;
    delta_prep_kernel<T><<<N, 32 * (units < 8 ? units : 8), 0, stream>>>(p);
    if (launch_status() != EMS_OK) return EMS_ERR_LAUNCH;
    if (N == rows) {
        delta_step_kernel<T><<<dim3((p.V + 127) / 128, p.H, rows), 128, 0, stream>>>(p);
        return launch_status();
    }
    // 16-byte copies of four floats where every row of the work buffer begins aligned
    p.vec_ok = p.D % 4 == 0 && p.V % 4 == 0 && p.work_ld % 4 == 0 && ((uintptr_t)p.work % 16) == 0;
    // Few lanes per column mean short reductions, and the lanes of a warp that hold the same rows of several
    // columns read q, k and g as one broadcast: 1.6 times the columns per SM and microsecond at D = 128.  But a
    // block then owns more columns, and a step of one or two requests leaves SMs idle; such steps spread a
    // column over more lanes (measured at 16 heads of 128 x 128, one prompt of 2048 tokens: 509 us over 128
    // blocks against 626 us over 64; at 32 heads the 256 blocks of the wide tiling are two waves, 1090 us).
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    // waves of blocks over the SMs, the narrow tiling's wave taken as a quarter longer
    auto narrow = [&](int cols_narrow) {
        const long long bn = (long long)rows * p.H * ((p.V + cols_narrow - 1) / cols_narrow);
        const long long bw = (long long)rows * p.H * ((p.V + cols_narrow / 2 - 1) / (cols_narrow / 2));
        return 5 * ((bn + sms - 1) / sms) < 4 * ((bw + sms - 1) / sms);
    };
    if (p.D <= 32) return launch_delta_as<T, 4, 8>(p, rows, stream);
    if (p.D <= 64) {
        if (narrow(DR_WARPS * 4 * DR_CPL)) return launch_delta_as<T, 8, 8>(p, rows, stream);
        return launch_delta_as<T, 4, 16>(p, rows, stream);
    }
    if (p.D <= 128) {
        if (narrow(DR_WARPS * 2 * DR_CPL)) return launch_delta_as<T, 8, 16>(p, rows, stream);
        return launch_delta_as<T, 4, 32>(p, rows, stream);
    }
    if (narrow(DR_WARPS * 2 * DR_CPL)) return launch_delta_as<T, 16, 16>(p, rows, stream);
    return launch_delta_as<T, 8, 32>(p, rows, stream);
}

// ---------------------------------------------------------------------------------------
// dt = softplus(x[t, h] + bias[h]);  a[t, h] = exp(-exp(a_log[h]) dt);  b[t, h] = dt

template <typename T>
__global__ void ssm_gates_kernel(const T* __restrict__ x, long long ldx, const void* __restrict__ bias,
                                 const void* __restrict__ a_log, int p_dtype, float* __restrict__ a,
                                 float* __restrict__ b, int N, int H) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N * H) return;
    const int t = i / H, h = i % H;
    const float dt = d_softplus(to_f32<T>(x[(size_t)t * ldx + h]) + load_any(bias, p_dtype, h));
    a[i] = expf(-expf(load_any(a_log, p_dtype, h)) * dt);
    b[i] = dt;
}

// y = (o + skip[h] act(x)) * silu(z);  out = y / rms_group(y) * w.  One warp per (token, group), or a
// block when a group is long.  o: float [N, C]; x, z: column ranges of wider buffers; head h owns the
// columns [h * hv, (h + 1) * hv).
template <typename T, bool BLOCK>
__global__ void gate_group_norm_kernel(const float* __restrict__ o, const T* __restrict__ x, long long ldx, int x_act,
                                       const void* __restrict__ skip, const T* __restrict__ z, long long ldz,
                                       const void* __restrict__ w, int w_dtype, T* __restrict__ out, int N, int C,
                                       int groups, int hv, float eps) {
    __shared__ float red[33];
    const int gs = C / groups;
    int unit, lane, width;
    if (BLOCK) { unit = blockIdx.x; lane = threadIdx.x; width = blockDim.x; }
    else { unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); lane = threadIdx.x & 31; width = 32; }
    if (unit >= N * groups) return;
    const int tok = unit / groups, g = unit % groups;
    auto value = [&](int ch) {
        float y = o[(size_t)tok * C + ch];
        if (skip) {
            const float xv = to_f32<T>(x[(size_t)tok * ldx + ch]);
            y = fmaf(load_any(skip, w_dtype, ch / hv), x_act ? d_silu(xv) : xv, y);
        }
        if (z) y *= d_silu(to_f32<T>(z[(size_t)tok * ldz + ch]));
        return y;
    };
    // (a thread's first eight values stay in registers between the two passes)
    constexpr int KEEP = 8;
    float kept[KEEP];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
        const int c = lane + i * width;
        kept[i] = c < gs ? value(g * gs + c) : 0.f;
        ss = fmaf(kept[i], kept[i], ss);
    }
    for (int c = lane + KEEP * width; c < gs; c += width) {
        const float y = value(g * gs + c);
        ss = fmaf(y, y, ss);
    }
    ss = BLOCK ? block_sum(ss, red) : warp_sum(ss);
    const float r = rsqrtf(ss / gs + eps);
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
        const int c = lane + i * width;
        if (c < gs) {
            const int ch = g * gs + c;
            out[(size_t)tok * C + ch] = from_f32<T>(kept[i] * r * load_any(w, w_dtype, ch));
        }
    }
    for (int c = lane + KEEP * width; c < gs; c += width) {
        const int ch = g * gs + c;
        out[(size_t)tok * C + ch] = from_f32<T>(value(ch) * r * load_any(w, w_dtype, ch));
    }
}

}  // namespace ems

using namespace ems;

EMS_EXPORT int ems_add_scaled_norm2(const void* d0, const void* d1, const void* d2, float s0, float s1, float s2,
                                    float* residual, const void* g1, const void* g2, int g_dtype, float gain_offset,
                                    float eps, void* out1, void* out2, int dtype, int n, int C, cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    if (C <= 0 || (out1 && !g1) || (out2 && !g2)) return EMS_ERR_SHAPE;
    int th = 32;
    while (th < 256 && th * 4 < C) th <<= 1;
    if (dtype == EMS_F32)
        add_scaled_norm2_kernel<float><<<n, th, 0, stream>>>((const float*)d0, (const float*)d1, (const float*)d2, s0, s1,
                                                             s2, residual, g1, g2, g_dtype, gain_offset, eps,
                                                             (float*)out1, (float*)out2, C);
    else if (dtype == EMS_BF16)
        add_scaled_norm2_kernel<bf16><<<n, th, 0, stream>>>((const bf16*)d0, (const bf16*)d1, (const bf16*)d2, s0, s1, s2,
                                                            residual, g1, g2, g_dtype, gain_offset, eps, (bf16*)out1,
                                                            (bf16*)out2, C);
    else
        return EMS_ERR_DTYPE;
    return launch_status();
}

EMS_EXPORT int ems_stream_norm(float* residual, const void* gain, int g_dtype, float gain_offset, float eps, int n,
                               int C, cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    if (C <= 0) return EMS_ERR_SHAPE;
    int th = 32;
    while (th < 256 && th * 4 < C) th <<= 1;
    stream_norm_kernel<<<n, th, 0, stream>>>(residual, gain, g_dtype, gain_offset, eps, C);
    return launch_status();
}

EMS_EXPORT int ems_softcap(float* x, long long n, float cap, cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    if (!(cap > 0.f)) return EMS_ERR_SHAPE;
    const long long blocks = (n + 255) / 256;
    softcap_kernel<<<(unsigned)(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, stream>>>(x, (size_t)n, cap);
    return launch_status();
}

EMS_EXPORT int ems_delta_recurrence(const void* q, long long ldq, const void* k, long long ldk, const void* v,
                                    long long ldv, const void* beta, long long ldb, int dtype, int act, int unit,
                                    float unit_eps, float q_scale, const float* g_raw, const void* g_bias,
                                    const void* a_log, int p_dtype, float* state, const int* slots, const int* cu_q,
                                    int rows, int N, int H, int HK, int D, int V, float* out, float* work,
                                    long long work_floats, cudaStream_t stream) {
    if (rows <= 0 || N <= 0) return EMS_OK;
    if (H <= 0 || HK <= 0 || H % HK || D <= 0 || D > 256 || V <= 0 || H > 65535 || rows > 65535) return EMS_ERR_SHAPE;
    // a row of the work buffer: q | k | g | v | k.q | beta, rounded up to a multiple of four floats
    const int work_ld = (2 * HK * D + H * D + H * V + HK + H + 3) / 4 * 4;
    if (!work || work_floats < (long long)N * work_ld) return EMS_ERR_SCRATCH;
    DeltaParams p;
    p.q = q; p.k = k; p.v = v; p.ldq = ldq; p.ldk = ldk; p.ldv = ldv; p.beta = beta; p.ldb = ldb; p.g_raw = g_raw;
    p.g_bias = g_bias; p.a_log = a_log; p.p_dtype = p_dtype; p.state = state; p.slots = slots; p.cu_q = cu_q;
    p.out = out; p.H = H; p.HK = HK; p.D = D; p.V = V; p.act = act; p.unit = unit; p.q_scale = q_scale;
    p.unit_eps = unit_eps; p.work = work; p.work_ld = work_ld; p.vec_ok = 0;
    if (dtype == EMS_F32) return launch_delta<float>(p, rows, N, stream);
    if (dtype == EMS_BF16) return launch_delta<bf16>(p, rows, N, stream);
    return EMS_ERR_DTYPE;
}

// floats of the work buffer that ems_delta_recurrence needs for N tokens
EMS_EXPORT long long ems_delta_work_floats(int N, int H, int HK, int D, int V) {
    return (long long)N * ((2 * HK * D + H * D + H * V + HK + H + 3) / 4 * 4);
}

EMS_EXPORT int ems_ssm_gates(const void* x, long long ldx, int dtype, const void* bias, const void* a_log, int p_dtype,
                             float* a, float* b, int N, int H, cudaStream_t stream) {
    if (N <= 0) return EMS_OK;
    if (H <= 0) return EMS_ERR_SHAPE;
    const unsigned blocks = (unsigned)(((long long)N * H + 255) / 256);
    if (dtype == EMS_F32)
        ssm_gates_kernel<float><<<blocks, 256, 0, stream>>>((const float*)x, ldx, bias, a_log, p_dtype, a, b, N, H);
    else if (dtype == EMS_BF16)
        ssm_gates_kernel<bf16><<<blocks, 256, 0, stream>>>((const bf16*)x, ldx, bias, a_log, p_dtype, a, b, N, H);
    else
        return EMS_ERR_DTYPE;
    return launch_status();
}

EMS_EXPORT int ems_gate_group_norm(const float* o, const void* x, long long ldx, int x_act, const void* skip,
                                   const void* z, long long ldz, const void* w, int w_dtype, void* out, int dtype,
                                   int N, int C, int groups, int hv, float eps, cudaStream_t stream) {
    if (N <= 0) return EMS_OK;
    if (groups <= 0 || C % groups || hv <= 0 || C % hv || (skip && !x)) return EMS_ERR_SHAPE;
    const int gs = C / groups;
    const long long units = (long long)N * groups;
#define EMS_LAUNCH_GGN(T)                                                                                          \
    do {                                                                                                           \
        if (gs > 256)                                                                                              \
            gate_group_norm_kernel<T, true><<<(unsigned)units, gs > 1024 ? 256 : 128, 0, stream>>>(                \
                o, (const T*)x, ldx, x_act, skip, (const T*)z, ldz, w, w_dtype, (T*)out, N, C, groups, hv, eps);   \
        else                                                                                                       \
            gate_group_norm_kernel<T, false><<<(unsigned)((units + 3) / 4), 128, 0, stream>>>(                     \
                o, (const T*)x, ldx, x_act, skip, (const T*)z, ldz, w, w_dtype, (T*)out, N, C, groups, hv, eps);   \
    } while (0)
    if (dtype == EMS_F32) EMS_LAUNCH_GGN(float);
    else if (dtype == EMS_BF16) EMS_LAUNCH_GGN(bf16);
    else return EMS_ERR_DTYPE;
#undef EMS_LAUNCH_GGN
    return launch_status();
}
