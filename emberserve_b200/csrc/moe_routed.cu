// Routed experts: a router that scores all experts per token, the choice of the `top` best, and
// the experts' gated feed-forwards run as two grouped matrix products over the (token, choice)
// pairs sorted by expert.
//
//   route     z[t, :] are the router's logits (32-bit, computed by the caller);
//             s = softmax(z) over all experts; the `top` largest (ties: the lower index) are
//             chosen; their weights are the scores s as they are (renorm = 0) or divided by
//             their sum (renorm = 1).  With scoring = 1 the scores are sigmoid(z) instead, each
//             expert by itself.  With a correction vector c the choice is made by s + c while the
//             weights stay the scores s; the weights may be divided by (their sum + an epsilon) and
//             multiplied by a constant; experts at and past `plan_experts` get no tiles (they have
//             no weights: the combine step returns their input).  The same kernel counts the pairs per expert, lays the
//             pairs out expert by expert (perm) and cuts each expert's rows into tiles.
//   up        act[i, :] = f(x[token(i)] Wg[e]^T) * (x[token(i)] Wu[e]^T)   for sorted pair i of expert e
//   down      y[pair(i), :] = act[i, :] Wd[e]^T            (32-bit, in pair order)
//   combine   out[t, :] = sum_k weight[t, k] * y[t * top + k, :]   (k ascending: a fixed order)
//
// A row of a product is accumulated over K in a fixed order, whatever else is in its tile: a
// token's result does not depend on the batch.  Products accumulate in 32 bits: on the tensor
// cores in bfloat16 (mma.sync), on the CUDA cores in the true 32-bit path.
#include "common.cuh"

namespace ems {

constexpr int MOE_TM = 64, MOE_TN = 64, MOE_TK = 16;

// One warp chooses for one token: lane l holds the logits of experts l, l + 32, ... (up to 8 each,
// so up to 256 experts; more are chosen by one lane alone).  Ties go to the lower index.
struct MoeRoute {
    int top, renorm, scoring;
    const float* corr;   // [E] added to the scores for the choice only, or null
    float renorm_eps;    // joins the sum the chosen scores are divided by
    float scale;         // multiplies the weights
};

__device__ __forceinline__ void moe_choose_serial(const float* __restrict__ z, int E, const MoeRoute r,
                                                  int* __restrict__ ids, float* __restrict__ wts, int* counts) {
    const int top = r.top;
    float mx = -INFINITY;
    for (int e = 0; e < E; ++e) mx = fmaxf(mx, z[e]);
    float sum = 0.f;
    for (int e = 0; e < E; ++e) sum += expf(z[e] - mx);
    float chosen_sum = 0.f;
    for (int k = 0; k < top; ++k) {
        int best = -1;
        float bv = -INFINITY, bs = 0.f;
        for (int e = 0; e < E; ++e) {
            bool taken = false;
            for (int j = 0; j < k; ++j) taken |= ids[j] == e;
            if (taken) continue;
            const float sc = r.scoring ? 1.f / (1.f + expf(-z[e])) : expf(z[e] - mx) / sum;
            const float cv = r.corr ? sc + r.corr[e] : z[e];   // (without a correction the logits order the scores)
            if (best < 0 || cv > bv) {
                best = e;
                bv = cv;
                bs = sc;
            }
        }
        ids[k] = best;
        wts[k] = bs;
        chosen_sum += bs;
        atomicAdd(&counts[best], 1);
    }
    for (int k = 0; k < top; ++k) wts[k] = (r.renorm ? wts[k] / (chosen_sum + r.renorm_eps) : wts[k]) * r.scale;
}

__device__ __forceinline__ void moe_choose_warp(const float* __restrict__ z, int E, const MoeRoute r,
                                                int* __restrict__ ids, float* __restrict__ wts, int* counts) {
    const int lane = threadIdx.x & 31;
    const int top = r.top;
    if (E > 256) {
        if (lane == 0) moe_choose_serial(z, E, r, ids, wts, counts);
        return;
    }
    float v[8], sc[8];   // what orders the choice, and the score
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = lane + 32 * i;
        v[i] = e < E ? z[e] : -INFINITY;
        mx = fmaxf(mx, v[i]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (lane + 32 * i < E) sum += expf(v[i] - mx);
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = lane + 32 * i;
        sc[i] = e < E ? (r.scoring ? 1.f / (1.f + expf(-v[i])) : expf(v[i] - mx) / sum) : 0.f;
        if (r.corr && e < E) v[i] = sc[i] + r.corr[e];   // (without a correction the logits order the scores)
    }
    float chosen_sum = 0.f;
    unsigned taken = 0u;  // bit i: my expert lane + 32 i is chosen already
    for (int k = 0; k < top; ++k) {
        float bv = -INFINITY, bs = 0.f;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (lane + 32 * i < E && !((taken >> i) & 1u) && (bi == 0x7fffffff || v[i] > bv)) {
                bv = v[i];
                bs = sc[i];
                bi = lane + 32 * i;
            }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const float os = __shfl_xor_sync(0xffffffffu, bs, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) {
                bv = ov;
                bs = os;
                bi = oi;
            }
        }
        chosen_sum += bs;
        if (lane == 0) {
            ids[k] = bi;
            wts[k] = bs;
            atomicAdd(&counts[bi], 1);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (lane + 32 * i == bi) taken |= 1u << i;
    }
    __syncwarp();
    if (lane == 0)
        for (int k = 0; k < top; ++k) wts[k] = (r.renorm ? wts[k] / (chosen_sum + r.renorm_eps) : wts[k]) * r.scale;
}

// plan (int32): [0] number of tiles; [1 .. 1 + 3 * max_tiles) expert, first sorted row and row
// count of each tile.  One block.
__global__ void moe_route_kernel(const float* __restrict__ logits, int n, int E, const MoeRoute r,
                                 int* __restrict__ ids, float* __restrict__ wts, int* __restrict__ offsets,
                                 int* __restrict__ perm, int* __restrict__ plan, int max_tiles, int plan_experts) {
    const int top = r.top;
    extern __shared__ int sh[];
    int* counts = sh;       // [E]
    int* cursor = sh + E;   // [E]
    int* offs = sh + 2 * E; // [E + 1]
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int t = threadIdx.x >> 5; t < n; t += blockDim.x >> 5)
        moe_choose_warp(logits + (size_t)t * E, E, r, ids + (size_t)t * top, wts + (size_t)t * top, counts);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0, nt = 0;
        for (int e = 0; e < E; ++e) {
            offs[e] = run;
            offsets[e] = run;
            cursor[e] = 0;
            for (int r0 = 0; e < plan_experts && r0 < counts[e] && nt < max_tiles; r0 += MOE_TM, ++nt) {
                plan[1 + 3 * nt] = e;
                plan[2 + 3 * nt] = run + r0;
                plan[3 + 3 * nt] = min(MOE_TM, counts[e] - r0);
            }
            run += counts[e];
        }
        offs[E] = run;
        offsets[E] = run;
        plan[0] = nt;
    }
    __syncthreads();
    for (int t = threadIdx.x; t < n; t += blockDim.x)
        for (int k = 0; k < top; ++k) {
            const int e = ids[(size_t)t * top + k];
            perm[offs[e] + atomicAdd(&cursor[e], 1)] = t * top + k;
        }
}

// The same in three kernels for steps of many tokens: one warp per token chooses and counts
// (counts in global memory, zeroed before), one block lays out offsets and tiles, one thread per
// pair takes its place among its expert's rows.
__global__ void moe_choose_kernel(const float* __restrict__ logits, int n, int E, const MoeRoute r,
                                  int* __restrict__ ids, float* __restrict__ wts, int* __restrict__ counts) {
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t < n)
        moe_choose_warp(logits + (size_t)t * E, E, r, ids + (size_t)t * r.top, wts + (size_t)t * r.top, counts);
}

// offsets: [E + 1]; counts and cursor: [E] each (the cursors are set to zero here).  With align > 1
// every expert's rows start at a multiple of `align` (the rows between are nobody's), and big[m]
// names the expert of the m-th group of `align` rows, -1 where the group is not in use.
__global__ void moe_plan_kernel(int E, const int* __restrict__ counts, int* __restrict__ cursor,
                                int* __restrict__ offsets, int* __restrict__ plan, int max_tiles, int align,
                                int* __restrict__ big, int max_big, int plan_experts) {
    if (threadIdx.x != 0) return;
    int run = 0, nt = 0, nb = 0;
    for (int e = 0; e < E; ++e) {
        if (align > 1) run = (run + align - 1) / align * align;
        offsets[e] = run;
        cursor[e] = 0;
        if (big)
            for (int r0 = 0; r0 < counts[e] && nb < max_big; r0 += align) big[nb++] = e < plan_experts ? e : -1;
        for (int r0 = 0; e < plan_experts && r0 < counts[e] && nt < max_tiles; r0 += MOE_TM, ++nt) {
            plan[1 + 3 * nt] = e;
            plan[2 + 3 * nt] = run + r0;
            plan[3 + 3 * nt] = min(MOE_TM, counts[e] - r0);
        }
        run += counts[e];
    }
    offsets[E] = run;
    plan[0] = nt;
    if (big)
        for (; nb < max_big; ++nb) big[nb] = -1;
}

// xs[i, :] = x[perm[i] / top, :] for the sorted rows i that belong to a pair (perm[i] >= 0); K a
// multiple of 8, 16-byte aligned rows.
__global__ void moe_gather_kernel(const bf16* __restrict__ x, const int* __restrict__ perm, int top, int K,
                                  bf16* __restrict__ xs) {
    const int i = blockIdx.x;
    const int p = perm[i];
    if (p < 0) return;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(p / top) * K);
    uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)i * K);
    for (int c = threadIdx.x; c < K / 8; c += blockDim.x) dst[c] = src[c];
}

// inv (optional): the sorted row of every pair, the inverse of perm
__global__ void moe_scatter_kernel(const int* __restrict__ ids, int pairs, const int* __restrict__ offsets,
                                   int* __restrict__ cursor, int* __restrict__ perm, int* __restrict__ inv) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= pairs) return;
    const int e = ids[p];
    const int row = offsets[e] + atomicAdd(&cursor[e], 1);
    perm[row] = p;
    if (inv) inv[p] = row;
}

__device__ __forceinline__ float moe_activation(float g, int act) {
    if (act == 1) return fmaxf(g, 0.f);
    if (act == 2) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    if (act == 4) return 0.5f * g * (1.f + erff(g * 0.7071067811865476f));
    return g / (1.f + expf(-g));
}

// What the up product stores from the 32-bit sums cg (gate) and cu (up) of one output.  act 0..2:
// f(g) * u of the two sums rounded to the storage type, as a product that is stored and read again would
// be.  act 3, the capped form: with g = min(s * cg, limit) and u = clamp(s * cu, -limit, limit) it is
// g * sigmoid(alpha * g) * (u + 1), all in 32 bits; s is the row's factor on the expert's INPUT (1 without).
struct MoeAct {
    int act;
    float limit, alpha;
};
template <typename T>
__device__ __forceinline__ float moe_glu(float cg, float cu, float s, const MoeAct a) {
    if (a.act == 3) {
        const float g = fminf(s * cg, a.limit);
        const float u = fminf(fmaxf(s * cu, -a.limit), a.limit);
        return g / (1.f + expf(-a.alpha * g)) * (u + 1.f);
    }
    const float g = round_to<T>(s * cg), u = round_to<T>(s * cu);
    return moe_activation(g, a.act) * u;
}

// MODE 1 (gated up): A rows are x[perm[row] / top] (gathered), B = w[e] of shape [2 N, K]; the tile
//              computes gate and up columns side by side and stores f(gate) * up in sorted order.
// MODE 2 (plain up): A rows gathered likewise, B = w[e] of shape [N, K]; the tile stores f(sum) in
//              sorted order (an expert without a gate).
// MODE 0 (down): A rows are a[row] (sorted order), B = w[e] of shape [N, K]; the tile is stored at
//              rows perm[row] of a 32-bit output.
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_grouped_kernel(const T* __restrict__ a, const T* __restrict__ w, const int* __restrict__ perm,
                   const int* __restrict__ plan, int top, int N, int K, const MoeAct act, T* __restrict__ out_t,
                   float* __restrict__ out_f, const float* __restrict__ in_scale) {
    __shared__ float As[MOE_TK][MOE_TM + 4];
    __shared__ float Bs[MOE_TK][MOE_TN + 4];
    constexpr bool GLU = MODE == 1;
    __shared__ float Bu[GLU ? MOE_TK : 1][MOE_TN + 4];
    __shared__ int src_row[MOE_TM];
    const int tile = blockIdx.x;
    if (tile >= plan[0]) return;
    const int e = plan[1 + 3 * tile], row0 = plan[2 + 3 * tile], rows = plan[3 + 3 * tile];
    const int n0 = blockIdx.y * MOE_TN;
    const T* we = w + (size_t)e * (GLU ? 2 : 1) * N * K;
    for (int i = threadIdx.x; i < MOE_TM; i += blockDim.x)
        src_row[i] = i < rows ? (MODE != 0 ? perm[row0 + i] / top : row0 + i) : -1;
    __syncthreads();
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int lr = threadIdx.x / 4, lk = (threadIdx.x % 4) * 4;  // the loader's row and first column
    float cg[4][4], cu[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) cg[i][j] = cu[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += MOE_TK) {
        const int ar = src_row[lr];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            As[lk + j][lr] = (ar >= 0 && k < K) ? to_f32<T>(a[(size_t)ar * K + k]) : 0.f;
            const int nn = n0 + lr;
            const bool ok = nn < N && k < K;
            Bs[lk + j][lr] = ok ? to_f32<T>(we[(size_t)nn * K + k]) : 0.f;
            if (GLU) Bu[lk + j][lr] = ok ? to_f32<T>(we[(size_t)(N + nn) * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_TK; ++kk) {
            float av[4], bv[4], uv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                bv[j] = Bs[kk][tx * 4 + j];
                if (GLU) uv[j] = Bu[kk][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    cg[i][j] = fmaf(av[i], bv[j], cg[i][j]);
                    if (GLU) cu[i][j] = fmaf(av[i], uv[j], cu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = n0 + tx * 4 + j;
            if (c >= N) continue;
            if (GLU) {
                const float sc = in_scale ? in_scale[perm[row0 + r]] : 1.f;
                out_t[(size_t)(row0 + r) * N + c] = from_f32<T>(moe_glu<T>(cg[i][j], cu[i][j], sc, act));
            } else if (MODE == 2) {
                const float sc = in_scale ? in_scale[perm[row0 + r]] : 1.f;
                out_t[(size_t)(row0 + r) * N + c] = from_f32<T>(moe_activation(round_to<T>(sc * cg[i][j]), act.act));
            } else {
                out_f[(size_t)perm[row0 + r] * N + c] = round_to<T>(cg[i][j]);
            }
        }
    }
}


// ---------------------------------------------------------------------------------------
// The same two products on the tensor cores (bfloat16, mma.sync m16n8k16, float32 accumulators).
// A block computes 64 sorted rows x 128 weight rows through a three-stage cp.async ring of
// 64-column slices; the activations' rows are gathered through the pair list as they are copied.
// GLU: the 128 weight rows are 64 gate rows and the 64 up rows of the same outputs, and a warp
// holds both halves of its outputs, so the activation is applied in registers.

constexpr int MM_TM = 64, MM_TB = 128, MM_TK = 64, MM_PAD = 8, MM_STAGES = 3;
constexpr int MM_SMEM = MM_STAGES * (MM_TM + MM_TB) * (MM_TK + MM_PAD) * 2;  // bytes of the ring

__device__ __forceinline__ void mm_cp_async16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void mm_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void mm_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void mm_ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int MODE>
__global__ void __launch_bounds__(256)
moe_grouped_mma_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w, const int* __restrict__ perm,
                       const int* __restrict__ plan, int top, int N, int K, const MoeAct act, bf16* __restrict__ out_t,
                       float* __restrict__ out_f, const float* __restrict__ in_scale) {
    constexpr int LDS = MM_TK + MM_PAD;  // elements per shared-memory row
    extern __shared__ __align__(16) unsigned char mm_smem[];
    bf16* As = reinterpret_cast<bf16*>(mm_smem);      // [MM_STAGES][MM_TM][LDS]
    bf16* Bs = As + MM_STAGES * MM_TM * LDS;          // [MM_STAGES][MM_TB][LDS]
    __shared__ int src_row[MM_TM];
    constexpr bool GLU = MODE == 1;
    const int tile = blockIdx.x;
    if (tile >= plan[0]) return;
    const int e = plan[1 + 3 * tile], row0 = plan[2 + 3 * tile], rows = plan[3 + 3 * tile];
    constexpr int NOUT = GLU ? MM_TB / 2 : MM_TB;  // output columns of a block
    const int n0 = blockIdx.y * NOUT;
    const bf16* we = w + (size_t)e * (GLU ? 2 : 1) * N * K;
    for (int i = threadIdx.x; i < MM_TM; i += blockDim.x)
        src_row[i] = i < rows ? (MODE != 0 ? perm[row0 + i] / top : row0 + i) : -1;
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm = warp >> 2, wn = warp & 3;  // 2 x 4 warps: 32 rows x (GLU ? 16 + 16 : 32) weight rows each
    const uint32_t as_base = (uint32_t)__cvta_generic_to_shared(As);
    const uint32_t bs_base = (uint32_t)__cvta_generic_to_shared(Bs);
    const int ktiles = (K + MM_TK - 1) / MM_TK;

    auto load = [&](int kt, int stage) {
        const int k0 = kt * MM_TK;
#pragma unroll
        for (int i = 0; i < 2; ++i) {  // activations: 64 rows x 8 chunks of 16 bytes
            const int idx = threadIdx.x + i * 256;
            const int r = idx >> 3, c = (idx & 7) * 8;
            const int ar = src_row[r];
            const bool ok = ar >= 0 && k0 + c < K;
            mm_cp_async16(as_base + (uint32_t)(((stage * MM_TM + r) * LDS + c) * 2),
                          ok ? a + (size_t)ar * K + k0 + c : a, ok);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // weights: 128 rows x 8 chunks
            const int idx = threadIdx.x + i * 256;
            const int r = idx >> 3, c = (idx & 7) * 8;
            int nn;  // the weight row that lands in shared row r
            if (GLU) nn = r < NOUT ? n0 + r : N + n0 + (r - NOUT);
            else nn = n0 + r;
            const bool ok = (GLU ? (n0 + (r % NOUT) < N) : (nn < N)) && k0 + c < K;
            mm_cp_async16(bs_base + (uint32_t)(((stage * MM_TB + r) * LDS + c) * 2),
                          ok ? we + (size_t)nn * K + k0 + c : we, ok);
        }
    };

    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

    for (int s = 0; s < MM_STAGES - 1; ++s) {
        if (s < ktiles) load(s, s);
        mm_commit();
    }
    const int a_row = (lane & 7) + 8 * ((lane >> 3) & 1), a_col = 8 * (lane >> 4);
    const int b_row = (lane & 7) + 8 * (lane >> 4), b_col = 8 * ((lane >> 3) & 1);
    for (int kt = 0; kt < ktiles; ++kt) {
        mm_wait<MM_STAGES - 2>();
        __syncthreads();
        if (kt + MM_STAGES - 1 < ktiles) load(kt + MM_STAGES - 1, (kt + MM_STAGES - 1) % MM_STAGES);
        mm_commit();
        const int stage = kt % MM_STAGES;
#pragma unroll
        for (int kk = 0; kk < MM_TK; kk += 16) {
            uint32_t af[2][4], bf[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                mm_ldmatrix_x4(as_base + (uint32_t)(((stage * MM_TM + wm * 32 + i * 16 + a_row) * LDS + kk + a_col) * 2),
                               af[i]);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                // GLU: j = 0 the warp's 16 gate rows, j = 1 its 16 up rows; else 32 consecutive rows
                const int brow = GLU ? (j * NOUT + wn * 16) : (wn * 32 + j * 16);
                mm_ldmatrix_x4(bs_base + (uint32_t)(((stage * MM_TB + brow + b_row) * LDS + kk + b_col) * 2), bf[j]);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    mm_mma(acc[i][2 * j], af[i], bf[j][0], bf[j][1]);
                    mm_mma(acc[i][2 * j + 1], af[i], bf[j][2], bf[j][3]);
                }
        }
    }
    mm_wait<0>();
    const int g = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            const int r = wm * 32 + i * 16 + g + 8 * hrow;
            if (r >= rows) continue;
            if (GLU) {
                const float sc = in_scale ? in_scale[perm[row0 + r]] : 1.f;
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int x = 0; x < 2; ++x) {
                        const int c = n0 + wn * 16 + nt * 8 + 2 * tq + x;
                        if (c >= N) continue;
                        out_t[(size_t)(row0 + r) * N + c] = from_f32<bf16>(
                            moe_glu<bf16>(acc[i][nt][2 * hrow + x], acc[i][2 + nt][2 * hrow + x], sc, act));
                    }
            } else if (MODE == 2) {
                const float sc = in_scale ? in_scale[perm[row0 + r]] : 1.f;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int x = 0; x < 2; ++x) {
                        const int c = n0 + wn * 32 + nt * 8 + 2 * tq + x;
                        if (c < N)
                            out_t[(size_t)(row0 + r) * N + c] = from_f32<bf16>(
                                moe_activation(round_to<bf16>(sc * acc[i][nt][2 * hrow + x]), act.act));
                    }
            } else {
                float* dst = out_f + (size_t)perm[row0 + r] * N;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int x = 0; x < 2; ++x) {
                        const int c = n0 + wn * 32 + nt * 8 + 2 * tq + x;
                        if (c < N) dst[c] = round_to<bf16>(acc[i][nt][2 * hrow + x]);
                    }
            }
        }
}

static bool moe_mma_ok(const void* a, const void* w, int K) {
    return K % 8 == 0 && !(reinterpret_cast<uintptr_t>(a) & 15) && !(reinterpret_cast<uintptr_t>(w) & 15);
}

// wts may be null (every weight 1: the scores went into the experts' inputs); `extra` (optional, [n, H]) is
// added last: the output of an expert that every token uses.
// With `ids` and `x`, a choice whose expert is at or past `num_real` has no weights: its output is the token's input x[t].
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ wts, T* __restrict__ out,
                                   int top, int H, const T* __restrict__ extra, const int* __restrict__ ids,
                                   const T* __restrict__ x, int num_real) {
    const size_t t = blockIdx.x;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k) {
            const bool same = ids && ids[t * top + k] >= num_real;
            s = fmaf(wts ? wts[t * top + k] : 1.f, same ? to_f32<T>(x[t * H + c]) : y[(t * top + k) * H + c], s);
        }
        if (extra) s += to_f32<T>(extra[t * H + c]);
        out[t * H + c] = from_f32<T>(s);
    }
}

// out[t, :] = sum_k wts[t, k] * y[inv[t * top + k], :] for y in bfloat16 in the sorted layout (wts may be
// null: every weight 1), plus extra[t, :] (optional)
__global__ void moe_combine_rows_kernel(const bf16* __restrict__ y, const int* __restrict__ inv,
                                        const float* __restrict__ wts, bf16* __restrict__ out, int top, int H,
                                        const bf16* __restrict__ extra, const int* __restrict__ ids,
                                        const bf16* __restrict__ x, int num_real) {
    const size_t t = blockIdx.x;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k) {
            const bool same = ids && ids[t * top + k] >= num_real;   // an expert that returns its input
            s = fmaf(wts ? wts[t * top + k] : 1.f,
                     __bfloat162float(same ? x[t * H + c] : y[(size_t)inv[t * top + k] * H + c]), s);
        }
        if (extra) s += __bfloat162float(extra[t * H + c]);
        out[t * H + c] = __float2bfloat16_rn(s);
    }
}

// The same, eight columns per thread and 16 bytes per load (H a multiple of 8, 16-byte aligned rows); a token's
// choices are added in the same order.
__global__ void moe_combine_rows_vec_kernel(const bf16* __restrict__ y, const int* __restrict__ inv,
                                            const float* __restrict__ wts, bf16* __restrict__ out, int top, int H,
                                            const bf16* __restrict__ extra, const int* __restrict__ ids,
                                            const bf16* __restrict__ x, int num_real) {
    const size_t t = blockIdx.x;
    for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
        float s[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j] = 0.f;
        for (int k = 0; k < top; ++k) {
            const bool same = ids && ids[t * top + k] >= num_real;
            const bf16* src = same ? x + t * H + c : y + (size_t)inv[t * top + k] * H + c;
            const uint4 raw = *reinterpret_cast<const uint4*>(src);
            const bf16* e = reinterpret_cast<const bf16*>(&raw);
            const float w = wts ? wts[t * top + k] : 1.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j] = fmaf(w, __bfloat162float(e[j]), s[j]);
        }
        if (extra) {
            const uint4 raw = *reinterpret_cast<const uint4*>(extra + t * H + c);
            const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j] += __bfloat162float(e[j]);
        }
        uint4 packed;
        bf16* o = reinterpret_cast<bf16*>(&packed);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(s[j]);
        *reinterpret_cast<uint4*>(out + t * H + c) = packed;
    }
}

}  // namespace ems

using namespace ems;

EMS_EXPORT int ems_moe_combine_rows(const void* y, const int* inv, const float* wts, void* out, int n, int top, int H,
                                    const void* extra, const int* ids, const void* x, int num_real,
                                    cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    int th = 32;
    const uintptr_t bits = (uintptr_t)y | (uintptr_t)out | (uintptr_t)extra | (uintptr_t)x;
    if (H % 8 == 0 && (bits & 15) == 0) {
        while (th * 8 < H && th < 256) th <<= 1;
        moe_combine_rows_vec_kernel<<<n, th, 0, stream>>>((const bf16*)y, inv, wts, (bf16*)out, top, H,
                                                          (const bf16*)extra, x ? ids : nullptr, (const bf16*)x, num_real);
        return launch_status();
    }
    while (th < H && th < 256) th <<= 1;
    moe_combine_rows_kernel<<<n, th, 0, stream>>>((const bf16*)y, inv, wts, (bf16*)out, top, H, (const bf16*)extra,
                                                  x ? ids : nullptr, (const bf16*)x, num_real);
    return launch_status();
}

EMS_EXPORT int ems_moe_tile_rows() { return MOE_TM; }

// align > 1 (steps of more than 512 tokens only): every expert's sorted rows start at a multiple of
// `align`; perm (max_big * align entries) holds -1 for the rows between, and big[0 .. max_big) names
// the expert of every group of `align` rows (-1: not in use); inv (optional, same steps) receives the
// sorted row of every pair.
EMS_EXPORT int ems_moe_route(const float* logits, int n, int E, int top, int renorm, int* ids, float* wts,
                             int* offsets, int* perm, int* plan, int max_tiles, int align, int* big, int max_big,
                             int* inv, int scoring, const float* corr, float renorm_eps, float scale,
                             int plan_experts, cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    if (top < 1 || top > E || scoring < 0 || scoring > 1) return EMS_ERR_SHAPE;
    if (align < 1 || (align > 1 && (n <= 512 || !big || max_big < n * top / align + (E < n * top ? E : n * top))))
        return EMS_ERR_SHAPE;
    if (plan_experts <= 0 || plan_experts > E) plan_experts = E;   // (every expert has weights)
    const MoeRoute r{top, renorm, scoring, corr, renorm_eps, scale};
    const size_t smem = (size_t)(3 * E + 1) * sizeof(int);
    if (smem > 48 * 1024) return EMS_ERR_SHAPE;
    if (n > 512) {  // `offsets` holds [offsets (E + 1) | counts (E) | cursors (E)]
        int* counts = offsets + E + 1;
        int* cursor = counts + E;
        if (cudaMemsetAsync(counts, 0, (size_t)E * sizeof(int), stream) != cudaSuccess) return EMS_ERR_LAUNCH;
        moe_choose_kernel<<<(n + 7) / 8, 256, 0, stream>>>(logits, n, E, r, ids, wts, counts);
        if (align > 1 &&
            cudaMemsetAsync(perm, 0xFF, (size_t)max_big * align * sizeof(int), stream) != cudaSuccess)
            return EMS_ERR_LAUNCH;
        moe_plan_kernel<<<1, 32, 0, stream>>>(E, counts, cursor, offsets, plan, max_tiles, align,
                                              align > 1 ? big : nullptr, max_big, plan_experts);
        moe_scatter_kernel<<<(n * top + 255) / 256, 256, 0, stream>>>(ids, n * top, offsets, cursor, perm, inv);
        return launch_status();
    }
    int th = 32 * (n < 32 ? n : 32);  // a warp per token, up to 32 warps
    moe_route_kernel<<<1, th, smem, stream>>>(logits, n, E, r, ids, wts, offsets, perm, plan, max_tiles, plan_experts);
    return launch_status();
}

// act: 0 SiLU, 1 ReLU, 2 tanh-GELU, 3 the capped form (see MoeAct; `limit` and `alpha` are its constants);
// in_scale (optional, [pairs] float): the factor on the input of each (token, choice) pair's expert.
EMS_EXPORT int ems_moe_up(const void* x, const void* wgu, int dtype, const int* perm, const int* plan, int max_tiles,
                          int top, int ff, int K, int act_code, void* out, int impl, const float* in_scale,
                          float limit, float alpha, int gated, cudaStream_t stream) {
    if (max_tiles <= 0) return EMS_OK;
    if (act_code < 0 || act_code > 4 || (gated == 0 && act_code == 3)) return EMS_ERR_SHAPE;
    const MoeAct act{act_code, limit, alpha};
    if (!gated) {   // experts without a gate: wgu is [E, ff, K]
        if (dtype == EMS_BF16 && impl == 0 && moe_mma_ok(x, wgu, K)) {
            dim3 mg(max_tiles, (ff + MM_TB - 1) / MM_TB);
            cudaFuncSetAttribute(moe_grouped_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, MM_SMEM);
            moe_grouped_mma_kernel<2><<<mg, 256, MM_SMEM, stream>>>((const bf16*)x, (const bf16*)wgu, perm, plan, top, ff,
                                                                 K, act, (bf16*)out, nullptr, in_scale);
            return launch_status();
        }
        dim3 grid(max_tiles, (ff + MOE_TN - 1) / MOE_TN);
        if (dtype == EMS_F32)
            moe_grouped_kernel<float, 2><<<grid, 256, 0, stream>>>((const float*)x, (const float*)wgu, perm, plan, top,
                                                                   ff, K, act, (float*)out, nullptr, in_scale);
        else if (dtype == EMS_BF16)
            moe_grouped_kernel<bf16, 2><<<grid, 256, 0, stream>>>((const bf16*)x, (const bf16*)wgu, perm, plan, top,
                                                                  ff, K, act, (bf16*)out, nullptr, in_scale);
        else
            return EMS_ERR_DTYPE;
        return launch_status();
    }
    // impl: 0 the tensor-core kernel where it takes the case, 1 always the CUDA-core kernel
    if (dtype == EMS_BF16 && impl == 0 && moe_mma_ok(x, wgu, K)) {
        dim3 mg(max_tiles, (ff + MM_TB / 2 - 1) / (MM_TB / 2));
        cudaFuncSetAttribute(moe_grouped_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, MM_SMEM);
        moe_grouped_mma_kernel<1><<<mg, 256, MM_SMEM, stream>>>((const bf16*)x, (const bf16*)wgu, perm, plan, top, ff, K,
                                                             act, (bf16*)out, nullptr, in_scale);
        return launch_status();
    }
    dim3 grid(max_tiles, (ff + MOE_TN - 1) / MOE_TN);
    if (dtype == EMS_F32)
        moe_grouped_kernel<float, 1><<<grid, 256, 0, stream>>>((const float*)x, (const float*)wgu, perm, plan, top,
                                                                  ff, K, act, (float*)out, nullptr, in_scale);
    else if (dtype == EMS_BF16)
        moe_grouped_kernel<bf16, 1><<<grid, 256, 0, stream>>>((const bf16*)x, (const bf16*)wgu, perm, plan, top,
                                                                 ff, K, act, (bf16*)out, nullptr, in_scale);
    else
        return EMS_ERR_DTYPE;
    return launch_status();
}

EMS_EXPORT int ems_moe_down(const void* a, const void* wdown, int dtype, const int* perm, const int* plan,
                            int max_tiles, int H, int ff, float* y, int impl, cudaStream_t stream) {
    if (max_tiles <= 0) return EMS_OK;
    if (dtype == EMS_BF16 && impl == 0 && moe_mma_ok(a, wdown, ff)) {
        dim3 mg(max_tiles, (H + MM_TB - 1) / MM_TB);
        cudaFuncSetAttribute(moe_grouped_mma_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, MM_SMEM);
        moe_grouped_mma_kernel<0><<<mg, 256, MM_SMEM, stream>>>((const bf16*)a, (const bf16*)wdown, perm, plan, 1, H, ff,
                                                              MoeAct{0, 0.f, 0.f}, nullptr, y, nullptr);
        return launch_status();
    }
    dim3 grid(max_tiles, (H + MOE_TN - 1) / MOE_TN);
    if (dtype == EMS_F32)
        moe_grouped_kernel<float, 0><<<grid, 256, 0, stream>>>((const float*)a, (const float*)wdown, perm, plan, 1,
                                                                   H, ff, MoeAct{0, 0.f, 0.f}, nullptr, y, nullptr);
    else if (dtype == EMS_BF16)
        moe_grouped_kernel<bf16, 0><<<grid, 256, 0, stream>>>((const bf16*)a, (const bf16*)wdown, perm, plan, 1,
                                                                  H, ff, MoeAct{0, 0.f, 0.f}, nullptr, y, nullptr);
    else
        return EMS_ERR_DTYPE;
    return launch_status();
}

EMS_EXPORT int ems_moe_gather(const void* x, const int* perm, int rows, int top, int K, void* xs,
                              cudaStream_t stream) {
    if (rows <= 0) return EMS_OK;
    if (K % 8 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(xs) & 15)) return EMS_ERR_ALIGN;
    int th = 32;
    while (th < K / 8 && th < 256) th <<= 1;
    moe_gather_kernel<<<rows, th, 0, stream>>>((const bf16*)x, perm, top, K, (bf16*)xs);
    return launch_status();
}

EMS_EXPORT int ems_moe_combine(const float* y, const float* wts, void* out, int dtype, int n, int top, int H,
                               const void* extra, const int* ids, const void* x, int num_real, cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    int th = 32;
    while (th < H && th < 256) th <<= 1;
    if (dtype == EMS_F32) moe_combine_kernel<float><<<n, th, 0, stream>>>(y, wts, (float*)out, top, H, (const float*)extra, x ? ids : nullptr, (const float*)x, num_real);
    else if (dtype == EMS_BF16) moe_combine_kernel<bf16><<<n, th, 0, stream>>>(y, wts, (bf16*)out, top, H, (const bf16*)extra, x ? ids : nullptr, (const bf16*)x, num_real);
    else return EMS_ERR_DTYPE;
    return launch_status();
}
