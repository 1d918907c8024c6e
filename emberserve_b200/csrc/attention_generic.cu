// Paged causal grouped-query attention over block tables, for any mix of rows: prompt
// portions (many queries) beside single decoded tokens.  This is the generic kernel:
// 32-bit arithmetic on CUDA cores, storage type float or bfloat16, any head size that
// is a multiple of 16 up to 256, any number of heads and groups, any page size, an
// optional sliding window, optional split of the keys over several blocks (decode).
// It is the kernel of the true 32-bit path and the fallback of the bfloat16 path.
//
// Formulas: emberserve/attn/base.py:105-128 (scores = q.k / sqrt(D); key j visible to
// the query at position p iff j <= p; softmax over keys; out = P.V; query head h reads
// KV head h / groups), and the paged form emberserve/attn/paged_torch.py:87-98.  A
// window of W keys additionally hides keys j <= p - W.
//
// Work split: a block owns BQ = 8*RPW "rows" of one request and one KV head, where a
// row is (query token, query head of the group): row r -> token r / G, head r % G.  So
// the G query heads that share a KV head share every K/V tile that is staged in shared
// memory.  Keys are walked in tiles of 32 whose boundaries are multiples of 32 in
// absolute position: the order of additions for a query does not depend on how the
// prompt was cut or on what else is in the batch.
#include "attention_decode_mma.cuh"
#include "common.cuh"

namespace ems {

constexpr int BK = 32;         // keys per tile = lanes of a warp
constexpr int NWARPS = 8;      // 256 threads

struct AttnParams {
    const void* q;      // [N, q_stride] first nh*D columns are the (rotated) queries
    void* out;          // [N, nh*D]
    const void* kc;     // [pages, nkv, page_size, D]
    const void* vc;
    const int* bt;      // [B, bt_stride]
    const int* cu_q;    // [B+1]
    const int* starts;  // [B] tokens cached before this step
    float* part_o;      // [N*nh, splits, D]   unnormalised partial outputs
    float* part_ml;     // [N*nh, splits, 2]   (running max, running sum)
    long long q_stride;
    int bt_stride, page_size, nh, nkv, D, G, window, splits;
    float scale;
    // Beyond the plain causal form (all optional):
    int chunk = 0;                  // > 0: the query at p sees only keys j with j / chunk == p / chunk
    const float* sinks = nullptr;   // [nh] float: exp(sinks[h]) joins the softmax's denominator (no key, no value)
    const void* gate = nullptr;     // [N, gate_stride]: head h's output is multiplied by sigmoid(gate[n, h])
    long long gate_stride = 0;
    int keep = 0;                   // > 0: keys j < keep stay visible to every later query, whatever the window says
    int DV = 0;                     // numbers per value head (the caches may differ in their last dimension)
    // Values that were turned by their own position before they were cached: the sum over the values is
    // turned back by the query's position.  out_table: [positions, DV / 2, (cos, sin)]; pair i is
    // (i, i + DV / 2) or, with out_pairing 1, (2 i, 2 i + 1).
    const float* out_table = nullptr;
    int out_pairing = 0;
    const int* positions = nullptr; // [N] position of every token of the step (for the merge of key splits)
    float softcap = 0.f;            // > 0: a scaled score s becomes softcap * tanh(s / softcap) before the softmax
};

template <typename T, int VEC> struct VecLoad;
template <> struct VecLoad<float, 4> {
    static __device__ __forceinline__ void load(const float* p, float* dst) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
    }
};
template <> struct VecLoad<bf16, 8> {
    static __device__ __forceinline__ void load(const bf16* p, float* dst) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            dst[2 * i] = f.x; dst[2 * i + 1] = f.y;
        }
    }
};

template <typename T, int DCH, int RPW>
__global__ void __launch_bounds__(NWARPS * 32)
paged_attention_kernel(const AttnParams p) {
    constexpr int BQ = NWARPS * RPW;
    constexpr int VEC = 16 / sizeof(T);
    extern __shared__ float smem[];
    const int D = p.D, G = p.G, DV = p.DV;
    const int KST = D + 1;                       // K tile row stride (no bank conflicts)
    float* Qs = smem;                            // [BQ][D]
    float* Ks = Qs + BQ * D;                     // [BK][D+1]
    float* Vs = Ks + BK * KST;                   // [BK][DV]
    float* Ps = Vs + BK * DV;                    // [BQ][BK+1]

    const int b = blockIdx.z / p.splits, split = blockIdx.z % p.splits;
    const int hk = blockIdx.y;
    const int q0 = p.cu_q[b], qlen = p.cu_q[b + 1] - q0, start = p.starts[b];
    const int nrows = qlen * G;
    const int r0 = blockIdx.x * BQ;
    if (r0 >= nrows) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int tok_lo = r0 / G;
    const int tok_hi = min(nrows - 1, r0 + BQ - 1) / G;
    const int p_lo = start + tok_lo, p_hi = start + tok_hi;
    const int k_begin = first_visible(p_lo, p.window, p.chunk);
    const int k_end = p_hi + 1;
    const int kt0 = (k_begin / BK) * BK;
    const int keep = min(p.keep, k_begin);       // kept keys that the window of the block's first query has passed
    const int nhead = min((keep + BK - 1) / BK, kt0 / BK);
    const int ntiles = nhead + (k_end - kt0 + BK - 1) / BK;
    const int tiles_per_split = (ntiles + p.splits - 1) / p.splits;
    const int t_begin = split * tiles_per_split;
    const int t_end = min(ntiles, t_begin + tiles_per_split);

    const T* qg = reinterpret_cast<const T*>(p.q);
    const T* kc = reinterpret_cast<const T*>(p.kc);
    const T* vc = reinterpret_cast<const T*>(p.vc);

    // stage the queries of this block
    for (int idx = threadIdx.x * VEC; idx < BQ * D; idx += NWARPS * 32 * VEC) {
        const int r = idx / D, d = idx % D;
        const int gr = r0 + r;
        float tmp[VEC];
        if (gr < nrows) {
            const int tok = gr / G, head = hk * G + gr % G;
            VecLoad<T, VEC>::load(qg + (size_t)(q0 + tok) * p.q_stride + (size_t)head * D + d, tmp);
        } else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) tmp[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < VEC; ++i) Qs[r * D + d + i] = tmp[i];
    }

    float m[RPW], l[RPW], o[RPW][DCH];
    int qpos[RPW], qlo[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        m[r] = -INFINITY;
        l[r] = 0.f;
        const int gr = r0 + warp * RPW + r;
        qpos[r] = gr < nrows ? start + gr / G : -1;   // -1: no key is visible
        qlo[r] = gr < nrows ? first_visible(qpos[r], p.window, p.chunk) : 0;
#pragma unroll
        for (int c = 0; c < DCH; ++c) o[r][c] = 0.f;
    }

    for (int t = t_begin; t < t_end; ++t) {
        const int kt = tile_start(t, nhead, kt0, BK);
        __syncthreads();  // previous tile fully consumed (and Qs written, first time)
        for (int idx = threadIdx.x * VEC; idx < BK * D; idx += NWARPS * 32 * VEC) {
            const int j = idx / D, d = idx % D;
            const int key = kt + j;
            float kk[VEC];
            if ((key >= k_begin || key < keep) && key < k_end) {
                const int page = p.bt[(size_t)b * p.bt_stride + key / p.page_size];
                VecLoad<T, VEC>::load(kc + (((size_t)page * p.nkv + hk) * p.page_size + key % p.page_size) * D + d, kk);
            } else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) kk[i] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < VEC; ++i) Ks[j * KST + d + i] = kk[i];
        }
        for (int idx = threadIdx.x * VEC; idx < BK * DV; idx += NWARPS * 32 * VEC) {
            const int j = idx / DV, d = idx % DV;
            const int key = kt + j;
            float vv[VEC];
            if ((key >= k_begin || key < keep) && key < k_end) {
                const int page = p.bt[(size_t)b * p.bt_stride + key / p.page_size];
                VecLoad<T, VEC>::load(vc + (((size_t)page * p.nkv + hk) * p.page_size + key % p.page_size) * DV + d, vv);
            } else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) vv[i] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < VEC; ++i) Vs[j * DV + d + i] = vv[i];
        }
        __syncthreads();

        // scores: lane = key of the tile, RPW rows per warp
        float acc[RPW];
#pragma unroll
        for (int r = 0; r < RPW; ++r) acc[r] = 0.f;
        const float* krow = Ks + lane * KST;
        const float* qrow = Qs + warp * RPW * D;
#pragma unroll 4
        for (int d = 0; d < D; ++d) {
            const float kv = krow[d];
#pragma unroll
            for (int r = 0; r < RPW; ++r) acc[r] = fmaf(qrow[r * D + d], kv, acc[r]);
        }
        const int key = kt + lane;
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            const bool visible = key <= qpos[r] && (key >= qlo[r] || key < p.keep);
            float s = -INFINITY;
            if (visible) s = p.softcap > 0.f ? p.softcap * tanhf(acc[r] * p.scale / p.softcap) : acc[r] * p.scale;
            const float m_new = fmaxf(m[r], warp_max(s));
            const float pe = visible ? expf(s - m_new) : 0.f;
            const float alpha = m_new == -INFINITY ? 1.f : expf(m[r] - m_new);
            l[r] = l[r] * alpha + warp_sum(pe);
            m[r] = m_new;
#pragma unroll
            for (int c = 0; c < DCH; ++c) o[r][c] *= alpha;
            Ps[(warp * RPW + r) * (BK + 1) + lane] = pe;
        }
        __syncwarp();
        // out += P.V : lane = head dimension (d = lane + 32*c)
        for (int j = 0; j < BK; ++j) {
            float pj[RPW];
#pragma unroll
            for (int r = 0; r < RPW; ++r) pj[r] = Ps[(warp * RPW + r) * (BK + 1) + j];
#pragma unroll
            for (int c = 0; c < DCH; ++c) {
                const int d = lane + 32 * c;
                if (d < DV) {
                    const float vv = Vs[j * DV + d];
#pragma unroll
                    for (int r = 0; r < RPW; ++r) o[r][c] = fmaf(pj[r], vv, o[r][c]);
                }
            }
        }
        __syncwarp();
    }

    // write out
    const bool turn_back = p.out_table && p.splits == 1;
    if (turn_back) __syncthreads();  // every warp is through with the last tile: Vs holds the rows now ([BQ][DV], BQ <= BK)
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        const int gr = r0 + warp * RPW + r;
        if (gr >= nrows) continue;
        const int tok = gr / G, head = hk * G + gr % G;
        const size_t prow = (size_t)(q0 + tok) * p.nh + head;
        if (p.splits == 1) {
            T* dst = reinterpret_cast<T*>(p.out) + prow * DV;
            float inv = 1.0f / (p.sinks ? l[r] + expf(p.sinks[head] - m[r]) : l[r]);
            if (p.gate)
                inv *= 1.f / (1.f + expf(-to_f32<T>(reinterpret_cast<const T*>(p.gate)[(size_t)(q0 + tok) * p.gate_stride + head])));
            if (turn_back) {
                float* row = Vs + (size_t)(warp * RPW + r) * DV;
#pragma unroll
                for (int c = 0; c < DCH; ++c) {
                    const int d = lane + 32 * c;
                    if (d < DV) row[d] = o[r][c] * inv;
                }
                __syncwarp();
                const int half = DV / 2;
                const float* cs = p.out_table + (size_t)qpos[r] * half * 2;
                for (int i = lane; i < half; i += 32) {
                    const int ia = p.out_pairing ? 2 * i : i, ib = p.out_pairing ? 2 * i + 1 : i + half;
                    const float cc = cs[2 * i], sn = cs[2 * i + 1], u = row[ia], w = row[ib];
                    dst[ia] = from_f32<T>(u * cc + w * sn);
                    dst[ib] = from_f32<T>(w * cc - u * sn);
                }
                continue;
            }
#pragma unroll
            for (int c = 0; c < DCH; ++c) {
                const int d = lane + 32 * c;
                if (d < DV) dst[d] = from_f32<T>(o[r][c] * inv);
            }
        } else {
            float* dst = p.part_o + (prow * p.splits + split) * DV;
#pragma unroll
            for (int c = 0; c < DCH; ++c) {
                const int d = lane + 32 * c;
                if (d < DV) dst[d] = o[r][c];
            }
            if (lane == 0) {
                p.part_ml[(prow * p.splits + split) * 2] = m[r];
                p.part_ml[(prow * p.splits + split) * 2 + 1] = l[r];
            }
        }
    }
}

// Merge the partial results of the splits: out = sum_s o_s * exp(m_s - M) / sum_s l_s * exp(m_s - M)
// (emberserve/attn/paged_triton.py:185-208).  One block per (token, head); splits are
// added in index order.
constexpr int MERGE_MAX_SPLITS = 256;

template <typename T>
__global__ void attention_merge_kernel(const float* __restrict__ part_o,
                                       const float* __restrict__ part_ml, T* __restrict__ out,
                                       int splits, int D, const float* __restrict__ sinks, int nh,
                                       const T* __restrict__ gate, long long gate_stride,
                                       const float* __restrict__ out_table, int out_pairing,
                                       const int* __restrict__ positions) {
    pdl_prologue();
    __shared__ float weight[MERGE_MAX_SPLITS];
    __shared__ float red[33];
    __shared__ float row[256];  // the merged head before it is turned back (out_table; D <= 256)
    const size_t prow = blockIdx.x;
    const float* ml = part_ml + prow * splits * 2;
    // the splits' maxima and sums are read side by side (a thread per split), the partial
    // outputs a column per thread with the loads of several splits in flight
    float m_loc = -INFINITY;
    for (int s = threadIdx.x; s < splits; s += blockDim.x) m_loc = fmaxf(m_loc, ml[s * 2]);
    const float M = block_max(m_loc, red);
    float d_loc = 0.f;
    for (int s = threadIdx.x; s < splits; s += blockDim.x) {
        const float ms = ml[s * 2];
        const float f = ms == -INFINITY ? 0.f : expf(ms - M);
        weight[s] = f;
        d_loc += ml[s * 2 + 1] * f;
    }
    float inv = block_sum(d_loc, red);  // (block_sum synchronises: the weights are written)
    if (sinks) inv += expf(sinks[prow % nh] - M);
    inv = 1.0f / inv;
    if (gate) inv *= 1.f / (1.f + expf(-to_f32<T>(gate[(prow / nh) * gate_stride + prow % nh])));
    const float* po = part_o + prow * splits * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.f;
#pragma unroll 8
        for (int s = 0; s < splits; ++s) acc += po[(size_t)s * D + d] * weight[s];  // in split order
        if (out_table) row[d] = acc * inv;
        else out[prow * D + d] = from_f32<T>(acc * inv);
    }
    if (out_table) {
        __syncthreads();
        const int half = D / 2;
        const float* cs = out_table + (size_t)positions[prow / nh] * half * 2;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const int ia = out_pairing ? 2 * i : i, ib = out_pairing ? 2 * i + 1 : i + half;
            const float cc = cs[2 * i], sn = cs[2 * i + 1], u = row[ia], w = row[ib];
            out[prow * D + ia] = from_f32<T>(u * cc + w * sn);
            out[prow * D + ib] = from_f32<T>(w * cc - u * sn);
        }
    }
}

template <typename T, int DCH, int RPW>
int launch_attention(const AttnParams& p, int B, int max_q_len, cudaStream_t stream) {
    constexpr int BQ = NWARPS * RPW;
    const size_t smem = sizeof(float) * ((size_t)BQ * p.D + (size_t)BK * (p.D + 1) + (size_t)BK * p.DV +
                                         (size_t)BQ * (BK + 1));
    auto kernel = paged_attention_kernel<T, DCH, RPW>;
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return EMS_ERR_LAUNCH;
    }
    const long long tiles = ((long long)max_q_len * p.G + BQ - 1) / BQ;
    const long long gz = (long long)B * p.splits;
    if (tiles > 2147483647LL || p.nkv > 65535 || gz > 65535) return EMS_ERR_SHAPE;
    const dim3 grid((unsigned)tiles, (unsigned)p.nkv, (unsigned)gz);
    kernel<<<grid, NWARPS * 32, smem, stream>>>(p);
    return launch_status();
}

template <typename T, int RPW>
int dispatch_dch(const AttnParams& p, int B, int max_q_len, cudaStream_t stream) {
    switch ((p.DV + 31) / 32) {
        case 1: return launch_attention<T, 1, RPW>(p, B, max_q_len, stream);
        case 2: return launch_attention<T, 2, RPW>(p, B, max_q_len, stream);
        case 3: return launch_attention<T, 3, RPW>(p, B, max_q_len, stream);
        case 4: return launch_attention<T, 4, RPW>(p, B, max_q_len, stream);
        case 5: return launch_attention<T, 5, RPW>(p, B, max_q_len, stream);
        case 6: return launch_attention<T, 6, RPW>(p, B, max_q_len, stream);
        case 7: return launch_attention<T, 7, RPW>(p, B, max_q_len, stream);
        case 8: return launch_attention<T, 8, RPW>(p, B, max_q_len, stream);
    }
    return EMS_ERR_SHAPE;
}

template <typename T>
int run_attention(const AttnParams& p, int B, int N, int max_q_len, cudaStream_t stream) {
    // Few rows per request (decode, short portions): 8-row blocks waste less.
    const bool small = (long long)max_q_len * p.G <= 16;
    const int rc = small ? dispatch_dch<T, 1>(p, B, max_q_len, stream)
                         : dispatch_dch<T, 4>(p, B, max_q_len, stream);
    if (rc != EMS_OK || p.splits == 1) return rc;
    const int threads = p.DV >= 128 ? 128 : 64;
    attention_merge_kernel<T><<<(unsigned)((size_t)N * p.nh), threads, 0, stream>>>(
        p.part_o, p.part_ml, reinterpret_cast<T*>(p.out), p.splits, p.DV, p.sinks, p.nh,
        reinterpret_cast<const T*>(p.gate), p.gate_stride, p.out_table, p.out_pairing, p.positions);
    return launch_status();
}

}  // namespace ems

using namespace ems;

// Bytes of scratch that ems_paged_attention needs for `splits` > 1.
EMS_EXPORT long long ems_paged_attention_scratch_bytes(int N, int nh, int D, int splits) {
    if (splits <= 1) return 0;
    return (long long)N * nh * splits * (D + 2) * (long long)sizeof(float);
}

static int paged_attention_any(const void* q, long long q_stride, void* out, int dtype,
                               const void* kcache, const void* vcache, const int* block_tables,
                               int bt_stride, int page_size, const int* cu_q, const int* starts,
                               int B, int N, int nh, int nkv, int D, int window, float scale,
                               int max_q_len, int splits, void* scratch, long long scratch_bytes,
                               int impl, int chunk, const float* sinks, const void* gate, long long gate_stride,
                               int keep, int DV, const float* out_table, int out_pairing, const int* positions,
                               float softcap, cudaStream_t stream) {
    // impl: 0 = the fastest kernel that takes the case, 1 = the generic kernel, 2 = the
    // tcgen05 prompt kernel or an error, 3 = the mma.sync kernels where they take the case.
    if (B <= 0 || N <= 0) return EMS_OK;
    const int esize = dtype == EMS_F32 ? 4 : 2;
    // (rows of a head are moved 16 bytes at a time)
    if (DV <= 0) DV = D;
    if (D <= 0 || D % (16 / esize) || D > 256 || DV % (16 / esize) || DV > 256 || nkv <= 0 || nh % nkv ||
        page_size <= 0 || splits < 1 || splits > MERGE_MAX_SPLITS || chunk < 0 || keep < 0 ||
        (out_table && (DV % 2 || (splits > 1 && !positions))))
        return EMS_ERR_SHAPE;
    if (window <= 0 && chunk <= 0) keep = 0;  // every key is visible anyway
    // the tensor-core kernels know the plain causal form (and a window)
    const bool plain = chunk <= 0 && !sinks && !gate && keep == 0 && DV == D && !out_table && !(softcap > 0.f);
    if (!plain && impl == 2) return EMS_ERR_SHAPE;
    if ((q_stride * esize) % 16 || ((uintptr_t)q % 16) || ((uintptr_t)kcache % 16) || ((uintptr_t)vcache % 16))
        return EMS_ERR_ALIGN;
    AttnParams p;
    p.q = q; p.out = out; p.kc = kcache; p.vc = vcache; p.bt = block_tables; p.cu_q = cu_q;
    p.starts = starts; p.q_stride = q_stride; p.bt_stride = bt_stride; p.page_size = page_size;
    p.nh = nh; p.nkv = nkv; p.D = D; p.G = nh / nkv; p.window = window; p.splits = splits;
    p.scale = scale; p.part_o = nullptr; p.part_ml = nullptr;
    p.chunk = chunk; p.sinks = sinks; p.gate = gate; p.gate_stride = gate_stride;
    p.keep = keep; p.DV = DV; p.out_table = out_table; p.out_pairing = out_pairing; p.positions = positions;
    p.softcap = softcap > 0.f ? softcap : 0.f;
    if (splits > 1) {
        if (scratch == nullptr || scratch_bytes < ems_paged_attention_scratch_bytes(N, nh, DV, splits))
            return EMS_ERR_SCRATCH;
        p.part_o = reinterpret_cast<float*>(scratch);
        p.part_ml = p.part_o + (size_t)N * nh * splits * DV;
    }
    DecodeParams d;
    d.q = reinterpret_cast<const bf16*>(q); d.out = reinterpret_cast<bf16*>(out);
    d.kc = reinterpret_cast<const bf16*>(kcache); d.vc = reinterpret_cast<const bf16*>(vcache);
    d.bt = block_tables; d.cu_q = cu_q; d.starts = starts; d.part_o = p.part_o; d.part_ml = p.part_ml;
    d.q_stride = q_stride; d.bt_stride = bt_stride; d.page_size = page_size; d.nh = nh; d.nkv = nkv;
    d.G = p.G; d.window = window; d.splits = splits;
    d.scale_log2 = scale * 1.4426950408889634f;
    d.chunk = chunk; d.sinks = sinks; d.gate = reinterpret_cast<const bf16*>(gate); d.gate_stride = gate_stride;
    d.keep = keep; d.out_table = out_table; d.out_pairing = out_pairing; d.positions = positions;
    d.softcap = p.softcap; d.scale = scale;
    if (!plain) {
        // prompt portions on the tensor cores where the sizes allow; everything else on the generic kernel
        const bool mma_form = DV == D;
        if (!mma_form) {
            if (dtype == EMS_F32) return run_attention<float>(p, B, N, max_q_len, stream);
            if (dtype == EMS_BF16) return run_attention<bf16>(p, B, N, max_q_len, stream);
            return EMS_ERR_DTYPE;
        }
        if ((impl == 0 || impl == 3) && splits == 1 && max_q_len > 1 &&
            prefill_mma_supported(dtype, D, q_stride, q, out, kcache, vcache) && (gate_stride * 2) % 2 == 0)
            return run_prefill_mma_masked(d, B, D, max_q_len, stream);
        if ((impl == 0 || impl == 3) && max_q_len == 1 && N == B &&
            decode_mma_supported(dtype, D, p.G, q_stride, q, kcache, vcache)) {
            const int rc = run_decode_mma(d, B, D, stream);
            if (rc != EMS_OK || splits == 1) return rc;
            return launch_pdl(attention_merge_kernel<bf16>, dim3((unsigned)((size_t)N * nh)),
                              dim3(D >= 128 ? 128 : 64), 0, stream, (const float*)p.part_o, (const float*)p.part_ml,
                              reinterpret_cast<bf16*>(out), splits, D, sinks, nh, reinterpret_cast<const bf16*>(gate),
                              gate_stride, out_table, out_pairing, positions);
        }
        if (dtype == EMS_F32) return run_attention<float>(p, B, N, max_q_len, stream);
        if (dtype == EMS_BF16) return run_attention<bf16>(p, B, N, max_q_len, stream);
        return EMS_ERR_DTYPE;
    }
    // impl 2 asks for the tcgen05 prompt kernel whatever the length (tests); by default it takes
    // the portions whose longest request fills eight of its 256-row blocks per KV head, below
    // which the mma.sync kernel with its smaller tiles was measured to be as fast or faster.
    if ((impl == 2 || (impl == 0 && (long long)max_q_len * p.G >= 2048)) && splits == 1 && max_q_len > 1 &&
        prefill_tc05_supported(dtype, D, page_size, q_stride, q, out, kcache, vcache))
        return run_prefill_tc05(d, B, D, max_q_len, stream);
    if (impl == 2) return EMS_ERR_SHAPE;
    if ((impl == 0 || impl == 3) && splits == 1 && max_q_len > 1 &&
        prefill_mma_supported(dtype, D, q_stride, q, out, kcache, vcache))
        return run_prefill_mma(d, B, D, max_q_len, stream);
    if ((impl == 0 || impl == 3) && max_q_len == 1 && N == B &&
        decode_mma_supported(dtype, D, p.G, q_stride, q, kcache, vcache)) {
        const int rc = run_decode_mma(d, B, D, stream);
        if (rc != EMS_OK || splits == 1) return rc;
        return launch_pdl(attention_merge_kernel<bf16>, dim3((unsigned)((size_t)N * nh)), dim3(D >= 128 ? 128 : 64),
                          0, stream, (const float*)p.part_o, (const float*)p.part_ml, reinterpret_cast<bf16*>(out),
                          splits, D, (const float*)nullptr, nh, (const bf16*)nullptr, 0LL, (const float*)nullptr, 0,
                          (const int*)nullptr);
    }
    if (dtype == EMS_F32) return run_attention<float>(p, B, N, max_q_len, stream);
    if (dtype == EMS_BF16) return run_attention<bf16>(p, B, N, max_q_len, stream);
    return EMS_ERR_DTYPE;
}

EMS_EXPORT int ems_paged_attention(const void* q, long long q_stride, void* out, int dtype,
                                   const void* kcache, const void* vcache, const int* block_tables,
                                   int bt_stride, int page_size, const int* cu_q, const int* starts,
                                   int B, int N, int nh, int nkv, int D, int window, float scale,
                                   int max_q_len, int splits, void* scratch, long long scratch_bytes,
                                   int impl, cudaStream_t stream) {
    return paged_attention_any(q, q_stride, out, dtype, kcache, vcache, block_tables, bt_stride, page_size, cu_q,
                               starts, B, N, nh, nkv, D, window, scale, max_q_len, splits, scratch, scratch_bytes,
                               impl, 0, nullptr, nullptr, 0, 0, D, nullptr, 0, nullptr, 0.f, stream);
}

// The same with a chunk mask, a sink per head in the softmax's denominator, a sigmoid gate per
// (token, head) on the output, first keys that a window never hides (keep), value heads of another size
// than the key heads (DV; vcache is [pages, nkv, page_size, DV] and out [N, nh * DV]) and values that were
// turned by their positions when they were cached (out_table: the result is turned back by the query's
// position, positions[n] of token n); each is optional (0 / null).
EMS_EXPORT int ems_paged_attention_masked(const void* q, long long q_stride, void* out, int dtype,
                                          const void* kcache, const void* vcache, const int* block_tables,
                                          int bt_stride, int page_size, const int* cu_q, const int* starts,
                                          int B, int N, int nh, int nkv, int D, int window, int chunk,
                                          const float* sinks, const void* gate, long long gate_stride, float scale,
                                          int max_q_len, int splits, void* scratch, long long scratch_bytes,
                                          int impl, int keep, int DV, const float* out_table, int out_pairing,
                                          const int* positions, float softcap, cudaStream_t stream) {
    return paged_attention_any(q, q_stride, out, dtype, kcache, vcache, block_tables, bt_stride, page_size, cu_q,
                               starts, B, N, nh, nkv, D, window, scale, max_q_len, splits, scratch, scratch_bytes,
                               impl, chunk, sinks, gate, gate_stride, keep, DV, out_table, out_pairing, positions,
                               softcap, stream);
}

// ---------------------------------------------------------------------------------------
// The variant that allocates nothing (see no_alloc.h for the contract and for who needs
// it): the partial results of the splits go to a fixed array inside the library.
#include "no_alloc.h"

#include <mutex>

static __device__ __align__(256) unsigned char g_static_scratch[EMS_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_scratch_mutex;
void* g_static_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of g_static_scratch on the current device; taken once per device.  In
// host code the symbol's name is not that address, so it must go through the runtime.
void* static_scratch_address() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess) {
            cudaGetLastError();  // leave no sticky error behind for the caller's next check
            return nullptr;
        }
        g_static_scratch_ptr[dev] = ptr;
    }
    return g_static_scratch_ptr[dev];
}
}  // namespace

EMS_EXPORT long long ems_static_scratch_capacity(void) { return (long long)EMS_STATIC_SCRATCH_BYTES; }

EMS_EXPORT int ems_paged_attention_static_scratch(
    const void* q, long long q_stride, void* out, int dtype, const void* kcache, const void* vcache,
    const int* block_tables, int bt_stride, int page_size, const int* cu_q, const int* starts, int B,
    int N, int nh, int nkv, int D, int window, float scale, int max_q_len, int splits,
    cudaStream_t stream) {
    if (splits <= 1)
        return ems_paged_attention(q, q_stride, out, dtype, kcache, vcache, block_tables, bt_stride,
                                   page_size, cu_q, starts, B, N, nh, nkv, D, window, scale, max_q_len,
                                   1, nullptr, 0, /*impl: never the tcgen05 kernel, whose first use
                                   allocates a status word and tensor maps*/ 3, stream);
    if (N <= 0 || nh <= 0 || D <= 0) return B <= 0 || N <= 0 ? EMS_OK : EMS_ERR_SHAPE;
    const long long need = ems_paged_attention_scratch_bytes(N, nh, D, splits);
    if (need > (long long)EMS_STATIC_SCRATCH_BYTES) return EMS_ERR_SCRATCH;
    void* scratch = static_scratch_address();
    if (scratch == nullptr) return EMS_ERR_LAUNCH;
    return ems_paged_attention(q, q_stride, out, dtype, kcache, vcache, block_tables, bt_stride,
                               page_size, cu_q, starts, B, N, nh, nkv, D, window, scale, max_q_len,
                               splits, scratch, (long long)EMS_STATIC_SCRATCH_BYTES, 3, stream);
}

// Decode attention of a step whose rows all bring one token, fused with what precedes it in the
// unfused path: `qkv` holds the raw projections [q | k | v] of the rows; the kernel rotates q
// and k (rot = D, or 0 for none), writes the new key and value into the cache (write_kv) and
// attends.  With splits > 1, `scratch` holds the partials and the merge kernel follows.  bfloat16, head sizes
// 64 and 128, at most 16 query heads per KV head; anything else returns EMS_ERR_SHAPE.
EMS_EXPORT int ems_decode_attention_fused(const void* qkv, long long q_stride, void* out, void* kcache,
                                          void* vcache, const int* block_tables, int bt_stride, int page_size,
                                          const int* cu_q, const int* starts, int B, int nh, int nkv, int D,
                                          int window, float scale, const float* rope_table, int rot, int write_kv,
                                          int splits, void* scratch, long long scratch_bytes, cudaStream_t stream) {
    if (B <= 0) return EMS_OK;
    if (nkv <= 0 || nh % nkv || page_size <= 0 || splits < 1 || splits > MERGE_MAX_SPLITS ||
        (rot != 0 && rope_table == nullptr))
        return EMS_ERR_SHAPE;
    if (!decode_fused_supported(D, nh / nkv, rot, q_stride, qkv, kcache, vcache)) return EMS_ERR_SHAPE;
    DecodeParams d;
    d.q = reinterpret_cast<const bf16*>(qkv); d.out = reinterpret_cast<bf16*>(out);
    d.kc = reinterpret_cast<const bf16*>(kcache); d.vc = reinterpret_cast<const bf16*>(vcache);
    d.bt = block_tables; d.cu_q = cu_q; d.starts = starts; d.part_o = nullptr; d.part_ml = nullptr;
    d.q_stride = q_stride; d.bt_stride = bt_stride; d.page_size = page_size; d.nh = nh; d.nkv = nkv;
    d.G = nh / nkv; d.window = window; d.splits = splits;
    d.scale_log2 = scale * 1.4426950408889634f;
    d.rope_table = rope_table; d.rot = rot; d.fused = 1; d.write_kv = write_kv;
    if (splits > 1) {
        const long long need = (long long)B * nh * splits * (D + 2) * (long long)sizeof(float);
        if (scratch == nullptr || scratch_bytes < need) return EMS_ERR_SCRATCH;
        d.part_o = reinterpret_cast<float*>(scratch);
        d.part_ml = d.part_o + (size_t)B * nh * splits * D;
    }
    const int rc = run_decode_mma(d, B, D, stream);
    if (rc != EMS_OK || splits == 1) return rc;
    return launch_pdl(attention_merge_kernel<bf16>, dim3((unsigned)((size_t)B * nh)), dim3(D >= 128 ? 128 : 64), 0,
                      stream, (const float*)d.part_o, (const float*)d.part_ml, reinterpret_cast<bf16*>(out), splits, D,
                      (const float*)nullptr, nh, (const bf16*)nullptr, 0LL, (const float*)nullptr, 0,
                      (const int*)nullptr);
}
