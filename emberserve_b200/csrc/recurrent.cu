// Mixers that carry state of fixed size from token to token instead of a growing cache:
//
//  * a matrix memory per head, S_t = a_t S_(t-1) + b_t k_t v_t^T, read as o_t = S_t^T q_t.  With a
//    constant decay per head and b = 1 this is linear ("lightning") attention; with gates a_t, b_t
//    from an exponential-gating recurrence and a normaliser vector n_t = a_t n_(t-1) + b_t k_t it is
//    the matrix memory of the mLSTM (Beck et al., "xLSTM: Extended Long Short-Term Memory");
//  * the stabilised gates of that memory (ems_mlstm_gates);
//  * a gated diagonal recurrence per channel, S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t (the
//    real-gated linear recurrent unit of De et al., "Griffin: Mixing Gated Linear Recurrences with
//    Local Attention for Efficient Language Models");
//  * the norm-and-gate step that follows a memory read (ems_group_norm_gate).
//
// Everything that enters a recurrence is 32-bit: states, decays, gates, the products with the state.
// The projections q, k, v, u, y arrive in the activation type and are widened once.  A request's
// tokens are walked in order by the same code whether they come as a prompt, a portion or alone, so
// a position's result does not depend on the cut.  States live in slots [slot, ...] of a float
// tensor; a block reads the state of its request's slot, runs the step's tokens and writes it back.
#include "common.cuh"

namespace ems {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
// log(sigmoid(z)) = min(z, 0) - log(1 + exp(-|z|))
__device__ __forceinline__ float logsigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// input activations of the memory's q, k, v
#define EMS_IN_NONE 0
#define EMS_IN_SILU 1
__device__ __forceinline__ float in_act(float z, int act) { return act == EMS_IN_SILU ? z * sigmoid_f(z) : z; }

// ---------------------------------------------------------------------------------------
// matrix memory
//
// A block of 16 warps owns a group of columns of one head's [v | 1] (the column of ones carries the
// normaliser) for one request.  A column is shared by SL lanes (32, 16 or 8, by the head's rows D);
// lane s holds rows i * 4 SL + 4 s + e (e < 4, i < DPT / 4) of the column of S in registers, so that
// the lanes of a warp read a staged q or k row as consecutive float4 and the dot product with q
// closes with shuffles among those lanes, once per tile.  The step's tokens are staged in tiles: q (scaled) and k (times
// b_t) widened and passed through the activation once; rows past D are zero.  A tile's inputs are
// asked for, as they lie in memory, while the tile before is computed, and widened when staged.
// Per token a thread does DPT multiply-adds into S and DPT into the read; only S carries from token
// to token, and with four warps per scheduler the latencies of one warp hide behind the others.

constexpr int MR_WARPS = 16;

struct MatRecParams {
    const void* q; const void* k; const void* v;   // [N, ld*] views; head h begins at column h * D (h * V)
    long long ldq, ldk, ldv;
    const float* decay_head;    // [H] constant decay per head, or null
    const float* a;             // [N, H] decay of every token (used when decay_head is null)
    const float* b;             // [N, H] input scale of every token, or null (= 1)
    const float* denom_floor;   // [N, H] with the normaliser: denom = max(|n.q|, floor) + denom_eps
    float* denom;               // [N, H] out (normaliser only)
    float* state;               // [slots, H, head_stride]: S [D, V] then, with the normaliser, n [D]
    const int* slots;           // [rows]
    const int* cu_q;            // [rows + 1]
    float* out;                 // [N, H * V] float
    int H, D, V, head_stride, normaliser, act, vec_ok;
    int qk_rep = 1;             // heads that share one head of q and k: head h reads q / k head h / qk_rep
    float q_scale, denom_eps;
};

// four consecutive elements of a row as they lie in memory (one 8- or 16-byte load), widened later:
// a tile's loads are all issued before any of them is looked at
template <typename T> struct Raw4;
template <> struct Raw4<float> {
    typedef float4 type;
    static __device__ __forceinline__ float4 widen(const float4& r) { return r; }
};
template <> struct Raw4<bf16> {
    typedef uint2 type;
    static __device__ __forceinline__ float4 widen(const uint2& r) {
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
        return make_float4(lo.x, lo.y, hi.x, hi.y);
    }
};

template <typename T, int DPT, int SL, int TT, bool VEC>
__global__ void __launch_bounds__(MR_WARPS * 32) matrix_recurrence_kernel(const MatRecParams p) {
    constexpr int THREADS = MR_WARPS * 32;
    constexpr int DP = SL * DPT;                   // rows the block can hold (>= D)
    constexpr int WCOLS = 32 / SL;                 // columns per warp
    constexpr int COLS = MR_WARPS * WCOLS;         // columns per block
    constexpr int GROUPS = TT * (DP / 4);          // groups of four q / k rows per tile
    constexpr int GPT = (GROUPS + THREADS - 1) / THREADS;
    constexpr int VPT = (TT * COLS + THREADS - 1) / THREADS;
    extern __shared__ __align__(16) float smem[];
    const int D = p.D, V = p.V;
    float* qs = smem;                    // [TT][DP]
    float* ks = qs + TT * DP;            // [TT][DP]   (already times b_t)
    float* vs = ks + TT * DP;            // [TT][COLS]
    float* as = vs + TT * COLS;          // [TT] decay
    float* fs = as + TT;                 // [TT] floor of the denominator
    const int row = blockIdx.z, head = blockIdx.y;
    const int q0 = p.cu_q[row], qlen = p.cu_q[row + 1] - q0;
    if (qlen <= 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slice = lane & (SL - 1), colw = lane / SL;
    const int lcol = warp * WCOLS + colw;          // column inside the block
    const int col = blockIdx.x * COLS + lcol;      // column of [v | 1]
    const int ncols = V + (p.normaliser ? 1 : 0);
    const bool live = col < ncols;
    const bool is_norm = p.normaliser && col == V;
    float* st = p.state + ((size_t)p.slots[row] * p.H + head) * p.head_stride;

    float S[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = (i / 4) * (4 * SL) + 4 * slice + (i & 3);
        S[i] = (live && d < D) ? (is_norm ? st[(size_t)D * V + d] : st[(size_t)d * V + col]) : 0.f;
    }
    const T* qg = reinterpret_cast<const T*>(p.q) + (size_t)(head / p.qk_rep) * D;
    const T* kg = reinterpret_cast<const T*>(p.k) + (size_t)(head / p.qk_rep) * D;
    const T* vg = reinterpret_cast<const T*>(p.v) + (size_t)head * V;
    const float decay_const = p.decay_head ? p.decay_head[head] : 1.f;

    typedef typename Raw4<T>::type raw4;
    float4 rq[VEC ? 1 : GPT], rk[VEC ? 1 : GPT];   // the scalar path (heads that do not begin aligned) widens at once
    raw4 wq[VEC ? GPT : 1], wk[VEC ? GPT : 1];     // the aligned path keeps what it loaded and widens when it is staged
    float rb[GPT], ra = 1.f, rf = 0.f;
    T rv[VPT];
    auto ask = [&](int t0) {
        const int cnt = min(TT, qlen - t0);
#pragma unroll
        for (int g = 0; g < GPT; ++g) {
            const int idx = threadIdx.x + g * THREADS;
            const int t = idx / (DP / 4), d = (idx % (DP / 4)) * 4;
            const bool ok = idx < GROUPS && t < cnt && d < D;
            const size_t tok = (size_t)(q0 + (ok ? t0 + t : 0));
            if constexpr (VEC) {   // straight-line: every load is issued, groups out of range read the first row again
                const int dd = ok ? d : 0;
                wq[g] = *reinterpret_cast<const raw4*>(qg + tok * p.ldq + dd);
                wk[g] = *reinterpret_cast<const raw4*>(kg + tok * p.ldk + dd);
            } else {
                rq[g] = make_float4(0.f, 0.f, 0.f, 0.f);
                rk[g] = rq[g];
                if (ok) {
                    const T* qr = qg + tok * p.ldq + d;
                    const T* kr = kg + tok * p.ldk + d;
                    rq[g].x = to_f32<T>(qr[0]);
                    rk[g].x = to_f32<T>(kr[0]);
                    if (d + 1 < D) { rq[g].y = to_f32<T>(qr[1]); rk[g].y = to_f32<T>(kr[1]); }
                    if (d + 2 < D) { rq[g].z = to_f32<T>(qr[2]); rk[g].z = to_f32<T>(kr[2]); }
                    if (d + 3 < D) { rq[g].w = to_f32<T>(qr[3]); rk[g].w = to_f32<T>(kr[3]); }
                }
            }
            rb[g] = p.b ? p.b[tok * p.H + head] : 1.f;
        }
#pragma unroll
        for (int g = 0; g < VPT; ++g) {
            const int idx = threadIdx.x + g * THREADS;
            const int t = idx / COLS, gc = blockIdx.x * COLS + idx % COLS;
            const bool ok = idx < TT * COLS && t < cnt && gc < V;
            rv[g] = vg[(size_t)(q0 + (ok ? t0 + t : 0)) * p.ldv + (ok ? gc : 0)];
        }
        {
            const bool ok = (int)threadIdx.x < cnt;
            const size_t at = (size_t)(q0 + (ok ? t0 + (int)threadIdx.x : 0)) * p.H + head;
            ra = p.decay_head ? decay_const : p.a[at];
            rf = p.normaliser ? p.denom_floor[at] : 0.f;
        }
    };
    ask(0);
    for (int t0 = 0; t0 < qlen; t0 += TT) {
        const int cnt = min(TT, qlen - t0);
        __syncthreads();  // the tile before is consumed
#pragma unroll
        for (int g = 0; g < GPT; ++g) {
            const int idx = threadIdx.x + g * THREADS;
            if (idx < GROUPS) {
                const int t = idx / (DP / 4), d = (idx % (DP / 4)) * 4;
                const bool ok = t < cnt && d < D;   // (rows past D and tokens past the end are staged as zeros)
                const float qsc = ok ? p.q_scale : 0.f, bt = ok ? rb[g] : 0.f;
                float4 fq, fk;
                if constexpr (VEC) { fq = Raw4<T>::widen(wq[g]); fk = Raw4<T>::widen(wk[g]); }
                else { fq = rq[g]; fk = rk[g]; }
                const float4 qq = make_float4(in_act(fq.x, p.act) * qsc, in_act(fq.y, p.act) * qsc,
                                              in_act(fq.z, p.act) * qsc, in_act(fq.w, p.act) * qsc);
                const float4 kk = make_float4(in_act(fk.x, p.act) * bt, in_act(fk.y, p.act) * bt,
                                              in_act(fk.z, p.act) * bt, in_act(fk.w, p.act) * bt);
                *reinterpret_cast<float4*>(qs + t * DP + d) = qq;
                *reinterpret_cast<float4*>(ks + t * DP + d) = kk;
            }
        }
#pragma unroll
        for (int g = 0; g < VPT; ++g) {
            const int idx = threadIdx.x + g * THREADS;
            if (idx < TT * COLS) {
                const int gc = blockIdx.x * COLS + idx % COLS;
                float val = 0.f;
                if (idx / COLS < cnt) {
                    if (gc < V) val = in_act(to_f32<T>(rv[g]), p.act);
                    else if (p.normaliser && gc == V) val = 1.f;   // the column of ones
                }
                vs[idx] = val;
            }
        }
        if ((int)threadIdx.x < TT) {
            as[threadIdx.x] = (int)threadIdx.x < cnt ? ra : 1.f;
            fs[threadIdx.x] = rf;
        }
        __syncthreads();
        if (t0 + TT < qlen) ask(t0 + TT);   // in flight while this tile is computed
        // every token of the tile (tokens past the end are staged as "decay 1, nothing added"); a lane
        // keeps its share of each token's read, and the shares are summed over the SL lanes of a
        // column once per tile: log2(SL) rounds in which a lane hands one half of what it holds to
        // its partner and adds the partner's other half, 31 shuffles for 32 tokens instead of 160
        float acc[TT];
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            const float a = as[t];
            const float vj = vs[t * COLS + lcol];
            const float4* k4 = reinterpret_cast<const float4*>(ks + t * DP) + slice;
            const float4* q4 = reinterpret_cast<const float4*>(qs + t * DP) + slice;
            float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
#pragma unroll
            for (int i = 0; i < DPT / 4; ++i) {
                const float4 kk = k4[i * SL], qq = q4[i * SL];
                S[4 * i + 0] = fmaf(a, S[4 * i + 0], kk.x * vj);
                S[4 * i + 1] = fmaf(a, S[4 * i + 1], kk.y * vj);
                S[4 * i + 2] = fmaf(a, S[4 * i + 2], kk.z * vj);
                S[4 * i + 3] = fmaf(a, S[4 * i + 3], kk.w * vj);
                acc0 = fmaf(S[4 * i + 0], qq.x, acc0);
                acc1 = fmaf(S[4 * i + 1], qq.y, acc1);
                acc2 = fmaf(S[4 * i + 2], qq.z, acc2);
                acc3 = fmaf(S[4 * i + 3], qq.w, acc3);
            }
            acc[t] = (acc0 + acc1) + (acc2 + acc3);
        }
#pragma unroll
        for (int off = SL / 2, n = TT; off >= 1; off >>= 1, n >>= 1) {
            const bool upper = (lane & off) != 0;
#pragma unroll
            for (int j = 0; j < n / 2; ++j) {
                const float send = upper ? acc[j] : acc[j + n / 2];
                const float keep = upper ? acc[j + n / 2] : acc[j];
                acc[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
            }
        }
        // lane `slice` of a column now holds the tokens [slice * TT / SL, (slice + 1) * TT / SL) of the tile
        if (live) {
#pragma unroll
            for (int j = 0; j < TT / SL; ++j) {
                const int t = slice * (TT / SL) + j;
                if (t < cnt) {
                    const size_t tok = (size_t)(q0 + t0 + t);
                    if (is_norm) p.denom[tok * p.H + head] = fmaxf(fabsf(acc[j]), fs[t]) + p.denom_eps;
                    else p.out[tok * ((size_t)p.H * V) + (size_t)head * V + col] = acc[j];
                }
            }
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = (i / 4) * (4 * SL) + 4 * slice + (i & 3);
            if (d < D) {
                if (is_norm) st[(size_t)D * V + d] = S[i];
                else st[(size_t)d * V + col] = S[i];
            }
        }
    }
}

// A step in which every request brings one token: the state is read and written once and nothing
// else matters.  A thread owns a column of [v | 1] and walks its rows, so that the lanes of a warp
// touch consecutive floats of every row of S.
template <typename T>
__global__ void __launch_bounds__(128) matrix_step_kernel(const MatRecParams p) {
    __shared__ float qs[256], ks[256];
    const int D = p.D, V = p.V;
    const int tok = blockIdx.z, head = blockIdx.y;   // (row r brings token r)
    const float bt = p.b ? p.b[(size_t)tok * p.H + head] : 1.f;
    const T* qg = reinterpret_cast<const T*>(p.q) + (size_t)tok * p.ldq + (size_t)(head / p.qk_rep) * D;
    const T* kg = reinterpret_cast<const T*>(p.k) + (size_t)tok * p.ldk + (size_t)(head / p.qk_rep) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        qs[d] = in_act(to_f32<T>(qg[d]), p.act) * p.q_scale;
        ks[d] = in_act(to_f32<T>(kg[d]), p.act) * bt;
    }
    __syncthreads();
    const int col = blockIdx.x * blockDim.x + threadIdx.x;
    const int ncols = V + (p.normaliser ? 1 : 0);
    if (col >= ncols) return;
    const bool is_norm = p.normaliser && col == V;
    const float a = p.decay_head ? p.decay_head[head] : p.a[(size_t)tok * p.H + head];
    const float vj = is_norm ? 1.f : in_act(to_f32<T>(reinterpret_cast<const T*>(p.v)[(size_t)tok * p.ldv + (size_t)head * V + col]), p.act);
    float* st = p.state + ((size_t)p.slots[tok] * p.H + head) * p.head_stride;
    float* sp = is_norm ? st + (size_t)D * V : st + col;
    const size_t step = is_norm ? 1 : (size_t)V;
    float acc0 = 0.f, acc1 = 0.f;
    int d = 0;
    for (; d + 1 < D; d += 2) {
        const float s0 = fmaf(a, sp[d * step], ks[d] * vj), s1 = fmaf(a, sp[(d + 1) * step], ks[d + 1] * vj);
        sp[d * step] = s0;
        sp[(d + 1) * step] = s1;
        acc0 = fmaf(s0, qs[d], acc0);
        acc1 = fmaf(s1, qs[d + 1], acc1);
    }
    if (d < D) {
        const float s0 = fmaf(a, sp[d * step], ks[d] * vj);
        sp[d * step] = s0;
        acc0 = fmaf(s0, qs[d], acc0);
    }
    const float acc = acc0 + acc1;
    if (is_norm) p.denom[(size_t)tok * p.H + head] = fmaxf(fabsf(acc), p.denom_floor[(size_t)tok * p.H + head]) + p.denom_eps;
    else p.out[(size_t)tok * ((size_t)p.H * V) + (size_t)head * V + col] = acc;
}

template <typename T, int DPT, int SL, int TT>
static int launch_matrix_recurrence_as(const MatRecParams& p, int rows, cudaStream_t stream) {
    constexpr int COLS = MR_WARPS * (32 / SL);
    const int ncols = p.V + (p.normaliser ? 1 : 0);
    const dim3 grid((ncols + COLS - 1) / COLS, p.H, rows);
    const size_t smem = sizeof(float) * ((size_t)TT * (2 * SL * DPT + COLS) + 2 * TT);
    auto kernel = p.vec_ok ? matrix_recurrence_kernel<T, DPT, SL, TT, true> : matrix_recurrence_kernel<T, DPT, SL, TT, false>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return EMS_ERR_LAUNCH;
    kernel<<<grid, MR_WARPS * 32, smem, stream>>>(p);
    return launch_status();
}

template <typename T>
static int launch_matrix_recurrence(MatRecParams& p, int rows, int N, cudaStream_t stream) {
    // 8- or 16-byte loads of four q / k elements where every row and head begins aligned
    const int e = (int)sizeof(T);
    p.vec_ok = p.D % 4 == 0 && p.ldq % 4 == 0 && p.ldk % 4 == 0 && ((uintptr_t)p.q % (4 * e)) == 0 &&
               ((uintptr_t)p.k % (4 * e)) == 0;
    if (p.D > 256) return EMS_ERR_SHAPE;
    if (N == rows) {   // every request brings one token
        const int ncols = p.V + (p.normaliser ? 1 : 0);
        matrix_step_kernel<T><<<dim3((ncols + 127) / 128, p.H, rows), 128, 0, stream>>>(p);
        return launch_status();
    }
    if (p.D <= 32) return launch_matrix_recurrence_as<T, 4, 8, 32>(p, rows, stream);
    if (p.D <= 64) return launch_matrix_recurrence_as<T, 4, 16, 32>(p, rows, stream);
    if (p.D <= 128) return launch_matrix_recurrence_as<T, 4, 32, 32>(p, rows, stream);
    return launch_matrix_recurrence_as<T, 8, 32, 32>(p, rows, stream);
}

// ---------------------------------------------------------------------------------------
// the gates of the mLSTM: log input gate i = cap tanh(x_i / cap), log forget gate f =
// logsigmoid(cap tanh(x_f / cap)), running maximum m_t = max(f + m_(t-1), i) (m starts at 0 in a
// fresh slot), a_t = exp(f + m_(t-1) - m_t), b_t = exp(i - m_t), floor_t = exp(-m_t).
// One warp per (request, head): the lanes take 32 tokens' transcendental work side by side, and the
// maximum runs through them as a scan of the maps m -> max(f + m, i).

__global__ void mlstm_gates_kernel(const float* __restrict__ pre, const void* __restrict__ bias_i,
                                   const void* __restrict__ bias_f, int b_dtype, float cap,
                                   float* __restrict__ state, int head_stride, int m_offset,
                                   const int* __restrict__ slots, const int* __restrict__ cu_q, int rows, int H,
                                   float* __restrict__ a_out, float* __restrict__ b_out,
                                   float* __restrict__ floor_out) {
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= rows * H) return;
    const int row = unit / H, head = unit % H, lane = threadIdx.x & 31;
    const int q0 = cu_q[row], qlen = cu_q[row + 1] - q0;
    if (qlen <= 0) return;
    float* mp = state + ((size_t)slots[row] * H + head) * head_stride + m_offset;
    float m = *mp;
    const float bi = load_any(bias_i, b_dtype, head), bf = load_any(bias_f, b_dtype, head);
    for (int t0 = 0; t0 < qlen; t0 += 32) {
        const int cnt = min(32, qlen - t0);
        float ig = 0.f, fg = 0.f;
        if (lane < cnt) {
            const size_t tok = (size_t)(q0 + t0 + lane);
            const float xi = pre[tok * 2 * H + head] + bi, xf = pre[tok * 2 * H + H + head] + bf;
            ig = cap > 0.f ? cap * tanhf(xi / cap) : xi;
            fg = logsigmoid_f(cap > 0.f ? cap * tanhf(xf / cap) : xf);
        }
        // m_t = max(f_t + m_(t-1), i_t) is the map m -> max(F + m, I) with (F, I) = (f_t, i_t); maps
        // compose as (F1, I1) then (F2, I2) = (F1 + F2, max(I1 + F2, I2)): a scan over the lanes.
        // (A lane past the end holds the identity (0, -inf).)
        float F = lane < cnt ? fg : 0.f, I = lane < cnt ? ig : -INFINITY;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const float Fp = __shfl_up_sync(0xffffffffu, F, off), Ip = __shfl_up_sync(0xffffffffu, I, off);
            if (lane >= off) {
                I = fmaxf(Ip + F, I);
                F += Fp;
            }
        }
        const float after = fmaxf(F + m, I);
        float before = __shfl_up_sync(0xffffffffu, after, 1);
        if (lane == 0) before = m;
        m = __shfl_sync(0xffffffffu, after, cnt - 1);
        if (lane < cnt) {
            const size_t at = (size_t)(q0 + t0 + lane) * H + head;
            a_out[at] = expf(fg + before - after);
            b_out[at] = expf(ig - after);
            floor_out[at] = expf(-after);
        }
    }
    if (lane == 0) *mp = m;
}

// ---------------------------------------------------------------------------------------
// what follows a memory read: o / denom (per token and group, optional), RMS norm of each of
// `groups` equal consecutive parts of the row, gain, sigmoid gate.  out = rms(o / denom) * w * sigmoid(g).
// One warp per (token, group); a block per (token, group) when a group is long.

template <typename T, bool BLOCK>
__global__ void group_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ denom,
                                       const void* __restrict__ w, int w_dtype, const T* __restrict__ gate,
                                       long long ldg, T* __restrict__ out, int N, int C, int groups, float eps) {
    __shared__ float red[33];
    const int gs = C / groups;
    int unit, lane, width;
    if (BLOCK) { unit = blockIdx.x; lane = threadIdx.x; width = blockDim.x; }
    else { unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); lane = threadIdx.x & 31; width = 32; }
    if (unit >= N * groups) return;   // (whole warps, or the whole block, leave together)
    const int tok = unit / groups, g = unit % groups;
    const float inv_den = denom ? 1.f / denom[(size_t)tok * groups + g] : 1.f;
    const float* src = o + (size_t)tok * C + (size_t)g * gs;
    float ss = 0.f;
    for (int c = lane; c < gs; c += width) {
        const float x = src[c] * inv_den;
        ss = fmaf(x, x, ss);
    }
    ss = BLOCK ? block_sum(ss, red) : warp_sum(ss);
    const float r = rsqrtf(ss / gs + eps) * inv_den;
    for (int c = lane; c < gs; c += width) {
        const int ch = g * gs + c;
        float y = src[c] * r * load_any(w, w_dtype, ch);
        if (gate) y *= sigmoid_f(to_f32<T>(gate[(size_t)tok * ldg + ch]));
        out[(size_t)tok * C + ch] = from_f32<T>(y);
    }
}

// ---------------------------------------------------------------------------------------
// the gated diagonal recurrence.  Gate pre-activations arrive as [2, blocks, N, C / blocks] float (r
// then i; the layout that one batched product per gate over the blocks of a block-diagonal matrix
// leaves): r = sigmoid(pre_r + br), i = sigmoid(pre_i + bi), log a = -c r softplus(lam),
// S = a S + sqrt(1 - a^2) i u, out = S * gelu_tanh(y).
//
// A block owns 32 channels of one request and walks its tokens in tiles of 32.  Per tile: with a
// lane per channel the threads load the tile and compute (a, b, gate) of every (token, channel);
// through shared memory the tile is turned so that a warp owns a channel with a lane per token and
// the recurrence S_t = a_t S_(t-1) + b_t becomes a scan of affine maps over the lanes (five
// shuffle steps), continued from the carry of the tile before; turned back, the threads store
// S * gate with a lane per channel.  The next tile's loads are issued before the scan.

constexpr int LRU_T = 32;   // tokens per tile
constexpr int LRU_C = 16;   // channels per block
constexpr int LRU_W = 8;    // warps

template <typename T>
__global__ void __launch_bounds__(LRU_W * 32)
rglru_scan_kernel(const T* __restrict__ u, const float* __restrict__ pre, const void* __restrict__ br,
                  const void* __restrict__ bi, const void* __restrict__ lam, int p_dtype, const T* __restrict__ y,
                  long long ldy, int y_act, float cmul, float* __restrict__ state, const int* __restrict__ slots,
                  const int* __restrict__ cu_q, T* __restrict__ out, int N, int C, int blocks) {
    __shared__ float sa[LRU_T][LRU_C + 1], sb[LRU_T][LRU_C + 1], sg[LRU_T][LRU_C + 1], carry[LRU_C];
    const int row = blockIdx.y;
    const int q0 = cu_q[row], qlen = cu_q[row + 1] - q0;
    if (qlen <= 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // loading and storing: a thread owns a channel and every ROWS-th token of the tile
    constexpr int ROWS = LRU_W * 32 / LRU_C, PER = LRU_T / ROWS;
    const int lc = threadIdx.x % LRU_C, lt = threadIdx.x / LRU_C;
    const int c = blockIdx.x * LRU_C + lc;
    const bool has_c = c < C;
    const int bw = C / blocks;
    const int cc = has_c ? c : 0;
    const float rb = load_any(br, p_dtype, cc), ib = load_any(bi, p_dtype, cc);
    const float sp = cmul * softplus_f(load_any(lam, p_dtype, cc));
    const float* pr = pre + ((size_t)(cc / bw) * N + q0) * bw + cc % bw;   // the r gate; the i gate lies N * C further
    const size_t gate_i = (size_t)N * C;
    float* st = state + (size_t)slots[row] * C;
    if (threadIdx.x < LRU_C) carry[lc] = has_c ? st[c] : 0.f;

    float l_r[PER], l_i[PER], l_u[PER], l_y[PER];
    auto load_tile = [&](int t0) {
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int t = t0 + lt + j * ROWS;
            if (has_c && t < qlen) {
                const size_t tok = (size_t)(q0 + t);
                l_r[j] = pr[(size_t)t * bw];
                l_i[j] = pr[(size_t)t * bw + gate_i];
                l_u[j] = to_f32<T>(u[tok * C + c]);
                l_y[j] = to_f32<T>(y[tok * ldy + c]);
            }
        }
    };
    load_tile(0);
    for (int t0 = 0; t0 < qlen; t0 += LRU_T) {
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int tl = lt + j * ROWS;
            float a = 1.f, b = 0.f, g = 0.f;   // a token past the end leaves the state as it is
            if (has_c && t0 + tl < qlen) {
                const float r = sigmoid_f(l_r[j] + rb);
                const float ig = sigmoid_f(l_i[j] + ib);
                const float log_a = -sp * r;
                a = expf(log_a);
                b = sqrtf(-expm1f(2.f * log_a)) * ig * l_u[j];   // sqrt(1 - a^2) without the cancellation
                g = y_act ? gelu_tanh_f(l_y[j]) : l_y[j];
            }
            sa[tl][lc] = a;
            sb[tl][lc] = b;
            sg[tl][lc] = g;
        }
        __syncthreads();
        if (t0 + LRU_T < qlen) load_tile(t0 + LRU_T);   // in flight during the scan
        // a warp per channel, a lane per token
#pragma unroll
        for (int j = 0; j < LRU_C / LRU_W; ++j) {
            const int ch = warp + j * LRU_W;
            float A = sa[lane][ch], B = sb[lane][ch];
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const float Ap = __shfl_up_sync(0xffffffffu, A, off), Bp = __shfl_up_sync(0xffffffffu, B, off);
                if (lane >= off) {
                    B = fmaf(A, Bp, B);
                    A *= Ap;
                }
            }
            const float S = fmaf(A, carry[ch], B);
            sb[lane][ch] = S;
            __syncwarp();
            if (lane == 31) carry[ch] = S;
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int tl = lt + j * ROWS;
            if (has_c && t0 + tl < qlen) out[(size_t)(q0 + t0 + tl) * C + c] = from_f32<T>(sb[tl][lc] * sg[tl][lc]);
        }
        __syncthreads();
    }
    if (threadIdx.x < LRU_C && has_c) st[c] = carry[lc];
}

// A step in which every request brings one token: a thread owns (request, channel).
template <typename T>
__global__ void rglru_step_kernel(const T* __restrict__ u, const float* __restrict__ pre, const void* __restrict__ br,
                                  const void* __restrict__ bi, const void* __restrict__ lam, int p_dtype,
                                  const T* __restrict__ y, long long ldy, int y_act, float cmul,
                                  float* __restrict__ state, const int* __restrict__ slots, T* __restrict__ out,
                                  int N, int C, int blocks) {
    const int tok = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int bw = C / blocks;
    const size_t at = ((size_t)(c / bw) * N + tok) * bw + c % bw;
    const float r = sigmoid_f(pre[at] + load_any(br, p_dtype, c));
    const float ig = sigmoid_f(pre[at + (size_t)N * C] + load_any(bi, p_dtype, c));
    const float log_a = -cmul * softplus_f(load_any(lam, p_dtype, c)) * r;
    float* sp = state + (size_t)slots[tok] * C + c;
    const float S = fmaf(expf(log_a), *sp, sqrtf(-expm1f(2.f * log_a)) * ig * to_f32<T>(u[(size_t)tok * C + c]));
    *sp = S;
    float yy = to_f32<T>(y[(size_t)tok * ldy + c]);
    if (y_act) yy = gelu_tanh_f(yy);
    out[(size_t)tok * C + c] = from_f32<T>(S * yy);
}

}  // namespace ems

using namespace ems;

EMS_EXPORT int ems_matrix_recurrence(const void* q, long long ldq, const void* k, long long ldk, const void* v,
                                     long long ldv, int dtype, int act, float q_scale, const float* decay_head,
                                     const float* a, const float* b, const float* denom_floor, float denom_eps,
                                     float* denom, float* state, int head_stride, int normaliser, const int* slots,
                                     const int* cu_q, int rows, int N, int H, int D, int V, float* out,
                                     int qk_heads, cudaStream_t stream) {
    if (rows <= 0 || N <= 0) return EMS_OK;
    if (qk_heads <= 0) qk_heads = H;   // (every head has q and k of its own)
    if (H % qk_heads) return EMS_ERR_SHAPE;
    if (H <= 0 || D <= 0 || V <= 0 || (!decay_head && !a) || (normaliser && (!denom || !denom_floor)) ||
        head_stride < D * V + (normaliser ? D : 0) || H > 65535 || rows > 65535)
        return EMS_ERR_SHAPE;
    MatRecParams p;
    p.q = q; p.k = k; p.v = v; p.ldq = ldq; p.ldk = ldk; p.ldv = ldv; p.decay_head = decay_head; p.a = a; p.b = b;
    p.denom_floor = denom_floor; p.denom = denom; p.state = state; p.slots = slots; p.cu_q = cu_q; p.out = out;
    p.H = H; p.D = D; p.V = V; p.head_stride = head_stride; p.normaliser = normaliser; p.act = act;
    p.q_scale = q_scale; p.denom_eps = denom_eps; p.qk_rep = H / qk_heads;
    if (dtype == EMS_F32) return launch_matrix_recurrence<float>(p, rows, N, stream);
    if (dtype == EMS_BF16) return launch_matrix_recurrence<bf16>(p, rows, N, stream);
    return EMS_ERR_DTYPE;
}

EMS_EXPORT int ems_mlstm_gates(const float* pre, const void* bias_i, const void* bias_f, int b_dtype, float cap,
                               float* state, int head_stride, int m_offset, const int* slots, const int* cu_q,
                               int rows, int H, float* a_out, float* b_out, float* floor_out, cudaStream_t stream) {
    if (rows <= 0) return EMS_OK;
    if (H <= 0 || m_offset < 0 || m_offset >= head_stride) return EMS_ERR_SHAPE;
    const int warps = 4;
    mlstm_gates_kernel<<<(rows * H + warps - 1) / warps, warps * 32, 0, stream>>>(
        pre, bias_i, bias_f, b_dtype, cap, state, head_stride, m_offset, slots, cu_q, rows, H, a_out, b_out, floor_out);
    return launch_status();
}

EMS_EXPORT int ems_group_norm_gate(const float* o, const float* denom, const void* w, int w_dtype, const void* gate,
                                   long long ldg, void* out, int dtype, int N, int C, int groups, float eps,
                                   cudaStream_t stream) {
    if (N <= 0) return EMS_OK;
    if (groups <= 0 || C % groups) return EMS_ERR_SHAPE;
    const int gs = C / groups;
    const long long units = (long long)N * groups;
#define EMS_LAUNCH_GNG(T)                                                                                        \
    do {                                                                                                         \
        if (gs > 256)                                                                                            \
            group_norm_gate_kernel<T, true><<<(unsigned)units, gs > 1024 ? 256 : 128, 0, stream>>>(              \
                o, denom, w, w_dtype, (const T*)gate, ldg, (T*)out, N, C, groups, eps);                          \
        else                                                                                                     \
            group_norm_gate_kernel<T, false><<<(unsigned)((units + 3) / 4), 128, 0, stream>>>(                   \
                o, denom, w, w_dtype, (const T*)gate, ldg, (T*)out, N, C, groups, eps);                          \
    } while (0)
    if (dtype == EMS_F32) EMS_LAUNCH_GNG(float);
    else if (dtype == EMS_BF16) EMS_LAUNCH_GNG(bf16);
    else return EMS_ERR_DTYPE;
#undef EMS_LAUNCH_GNG
    return launch_status();
}

EMS_EXPORT int ems_rglru_scan(const void* u, const float* pre, const void* br, const void* bi, const void* lam,
                              int p_dtype, const void* y, long long ldy, int y_act, float cmul, float* state,
                              const int* slots, const int* cu_q, void* out, int dtype, int rows, int N, int C,
                              int blocks, cudaStream_t stream) {
    if (rows <= 0 || N <= 0) return EMS_OK;
    if (blocks <= 0 || C % blocks || rows > 65535) return EMS_ERR_SHAPE;
    if (N == rows) {   // every request brings one token (the state of a request is independent of its row's index)
        const dim3 sgrid((C + 127) / 128, rows);
        if (dtype == EMS_F32)
            rglru_step_kernel<float><<<sgrid, 128, 0, stream>>>((const float*)u, pre, br, bi, lam, p_dtype, (const float*)y,
                                                                ldy, y_act, cmul, state, slots, (float*)out, N, C, blocks);
        else if (dtype == EMS_BF16)
            rglru_step_kernel<bf16><<<sgrid, 128, 0, stream>>>((const bf16*)u, pre, br, bi, lam, p_dtype, (const bf16*)y,
                                                               ldy, y_act, cmul, state, slots, (bf16*)out, N, C, blocks);
        else
            return EMS_ERR_DTYPE;
        return launch_status();
    }
    const int th = LRU_W * 32;
    const dim3 grid((C + LRU_C - 1) / LRU_C, rows);
    if (dtype == EMS_F32)
        rglru_scan_kernel<float><<<grid, th, 0, stream>>>((const float*)u, pre, br, bi, lam, p_dtype, (const float*)y,
                                                          ldy, y_act, cmul, state, slots, cu_q, (float*)out, N, C,
                                                          blocks);
    else if (dtype == EMS_BF16)
        rglru_scan_kernel<bf16><<<grid, th, 0, stream>>>((const bf16*)u, pre, br, bi, lam, p_dtype, (const bf16*)y,
                                                         ldy, y_act, cmul, state, slots, cu_q, (bf16*)out, N, C,
                                                         blocks);
    else
        return EMS_ERR_DTYPE;
    return launch_status();
}
