// Small steps around mixers and feed-forwards:
//
//  * ems_unary_act: out = act(x) for an ungated feed-forward (relu, relu squared, tanh-GELU, SiLU);
//  * ems_qk_prep: what stands between the projections and attention over a paged cache when the
//    heads are rotated, optionally brought to unit RMS, and the values are either projected or the
//    keys themselves as projected (before rotation and norm);
//  * ems_norm_mean2: the mean of two branches, each RMS-normed over the model width with a gain.
//
// Rotation angles come from a table of (cos, sin) per position and pair (any factor on cos and sin
// is part of the table); statistics and rotations are 32-bit, only stored values are rounded.
#include "common.cuh"

namespace ems {

#define EMS_ACT_RELU 0
#define EMS_ACT_RELU2 1
#define EMS_ACT_GELU_TANH 2
#define EMS_ACT_SILU 3
#define EMS_ACT_GELU_ERF 4

__device__ __forceinline__ float unary_activation(float z, int act) {
    if (act == EMS_ACT_RELU) return fmaxf(z, 0.f);
    if (act == EMS_ACT_RELU2) { const float r = fmaxf(z, 0.f); return r * r; }
    if (act == EMS_ACT_GELU_TANH) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    if (act == EMS_ACT_GELU_ERF) return 0.5f * z * (1.f + erff(z * 0.7071067811865476f));
    return z / (1.f + expf(-z));
}

template <typename T>
__global__ void unary_act_kernel(const T* __restrict__ x, T* __restrict__ out, size_t n, int act) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    out[i] = from_f32<T>(unary_activation(to_f32<T>(x[i]), act));
}

// 16 bytes per thread and trip, where the buffers begin on a 16-byte boundary
template <typename T>
__global__ void unary_act_vec_kernel(const uint4* __restrict__ x, uint4* __restrict__ out, size_t nvec, int act) {
    constexpr int PER = 16 / sizeof(T);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
        uint4 v = x[i];
        T* e = reinterpret_cast<T*>(&v);
#pragma unroll
        for (int j = 0; j < PER; ++j) e[j] = from_f32<T>(unary_activation(to_f32<T>(e[j]), act));
        out[i] = v;
    }
}

// One block per token, one warp per head at a time (query heads, then key heads, then value heads).
// proj row: [q: nh*D | k: nkv*D | v: nkv*DV (absent when the values are the keys)].  q is rewritten in
// place.  A value head may be brought to unit RMS (v_normed) and turned by the token's position over its
// whole length (v_table: [positions, DV / 2, (cos, sin)], pairs as v_pairing says) before it is cached.
template <typename T>
__global__ void qk_prep_kernel(T* __restrict__ proj, long long ld, int nh, int nkv, int D,
                               const int* __restrict__ positions, const int* __restrict__ row_of_token,
                               const float* __restrict__ table, int rot, int pairing, int normed, float eps,
                               T* __restrict__ kc, T* __restrict__ vc, const int* __restrict__ bt, int bt_stride,
                               int page_size, int values_are_keys, int write_kv, int DV, int v_normed, float v_eps,
                               const float* __restrict__ v_table, int v_pairing, const void* __restrict__ q_gain,
                               const void* __restrict__ k_gain, int gain_dtype, int norm_first) {
    extern __shared__ float smem[];
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    float* buf = smem + (size_t)warp * (D > DV ? D : DV);
    const int pos = positions[t];
    const int half = rot / 2;
    const float* cs = table ? table + (size_t)pos * half * 2 : nullptr;
    T* rowp = proj + (size_t)t * ld;
    size_t cache_at = 0;
    if (write_kv) {
        const int page = bt[(size_t)row_of_token[t] * bt_stride + pos / page_size];
        cache_at = ((size_t)page * nkv) * page_size + pos % page_size;  // + hk * page_size, times D below
    }
    const int nvh = (values_are_keys || !write_kv) ? 0 : nkv;  // value heads that pass through this kernel
    for (int h = warp; h < nh + nkv + nvh; h += nwarps) {
        if (h >= nh + nkv) {  // a value head
            const int hv = h - nh - nkv;
            const T* src = rowp + (size_t)(nh + nkv) * D + (size_t)hv * DV;
            T* dst = vc + (cache_at + (size_t)hv * page_size) * DV;
            float ss = 0.f;
            for (int d = lane; d < DV; d += 32) {
                const float x = to_f32<T>(src[d]);
                buf[d] = x;
                ss = fmaf(x, x, ss);
            }
            const float r = v_normed ? rsqrtf(warp_sum(ss) / DV + v_eps) : 1.f;
            __syncwarp();
            if (v_table) {
                const int vh = DV / 2;
                const float* vcs = v_table + (size_t)pos * vh * 2;
                for (int i = lane; i < vh; i += 32) {
                    const int ia = v_pairing ? 2 * i : i, ib = v_pairing ? 2 * i + 1 : i + vh;
                    const float c = vcs[2 * i], s = vcs[2 * i + 1];
                    const float a = buf[ia] * r, b = buf[ib] * r;
                    dst[ia] = from_f32<T>(a * c - b * s);
                    dst[ib] = from_f32<T>(b * c + a * s);
                }
            } else {
                for (int d = lane; d < DV; d += 32) dst[d] = v_normed ? from_f32<T>(buf[d] * r) : src[d];
            }
            __syncwarp();
            continue;
        }
        const bool is_k = h >= nh;
        const int hk = h - nh;
        T* src = rowp + (size_t)h * D;
        T* kdst = is_k && write_kv ? kc + (cache_at + (size_t)hk * page_size) * D : nullptr;
        T* vdst = is_k && write_kv && values_are_keys ? vc + (cache_at + (size_t)hk * page_size) * D : nullptr;
        for (int d = lane; d < D; d += 32) {
            const T raw = src[d];
            buf[d] = to_f32<T>(raw);
            if (vdst) vdst[d] = raw;
        }
        __syncwarp();
        const void* gain = is_k ? k_gain : q_gain;   // [D], shared by the heads (optional)
        if (normed && norm_first) {   // the norm (with its gain) comes before the rotation
            float ss = 0.f;
            for (int d = lane; d < D; d += 32) ss = fmaf(buf[d], buf[d], ss);
            const float r0 = rsqrtf(warp_sum(ss) / D + eps);
            for (int d = lane; d < D; d += 32) buf[d] = buf[d] * r0 * (gain ? load_any(gain, gain_dtype, d) : 1.f);
            __syncwarp();
        }
        if (cs) {
            for (int i = lane; i < half; i += 32) {
                const int ia = pairing ? 2 * i : i, ib = pairing ? 2 * i + 1 : i + half;
                const float c = cs[2 * i], s = cs[2 * i + 1];
                const float a = buf[ia], b = buf[ib];
                buf[ia] = a * c - b * s;
                buf[ib] = b * c + a * s;
            }
            __syncwarp();
        }
        float r = 1.f;
        if (normed && !norm_first) {
            float ss = 0.f;
            for (int d = lane; d < D; d += 32) ss = fmaf(buf[d], buf[d], ss);
            r = rsqrtf(warp_sum(ss) / D + eps);
            if (gain) {
                for (int d = lane; d < D; d += 32) buf[d] *= load_any(gain, gain_dtype, d);
                __syncwarp();
            }
        }
        for (int d = lane; d < D; d += 32) {
            const T val = from_f32<T>(buf[d] * r);
            if (!is_k) src[d] = val;
            else if (kdst) kdst[d] = val;
        }
        __syncwarp();
    }
}

// out = 0.5 * (rms(a) * wa + rms(b) * wb), rows of width C; one block per row.
template <typename T>
__global__ void norm_mean2_kernel(const T* __restrict__ a, const T* __restrict__ b, const void* __restrict__ wa,
                                  const void* __restrict__ wb, int w_dtype, T* __restrict__ out, int C, float eps) {
    __shared__ float red[33];
    const size_t base = (size_t)blockIdx.x * C;
    float sa = 0.f, sb = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float x = to_f32<T>(a[base + c]), y = to_f32<T>(b[base + c]);
        sa = fmaf(x, x, sa);
        sb = fmaf(y, y, sb);
    }
    const float ra = rsqrtf(block_sum(sa, red) / C + eps);
    const float rb = rsqrtf(block_sum(sb, red) / C + eps);
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float x = to_f32<T>(a[base + c]) * ra * load_any(wa, w_dtype, c);
        const float y = to_f32<T>(b[base + c]) * rb * load_any(wb, w_dtype, c);
        out[base + c] = from_f32<T>(0.5f * (x + y));
    }
}

}  // namespace ems

using namespace ems;

EMS_EXPORT int ems_unary_act(const void* x, void* out, int dtype, long long n, int act, cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    if (act < 0 || act > 4) return EMS_ERR_SHAPE;
    const int per = dtype == EMS_F32 ? 4 : 8;
    if ((dtype == EMS_F32 || dtype == EMS_BF16) && n % per == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        const size_t nvec = (size_t)(n / per);
        const unsigned vblocks = (unsigned)((nvec + 255) / 256 < 148 * 16 ? (nvec + 255) / 256 : 148 * 16);
        if (dtype == EMS_F32)
            unary_act_vec_kernel<float><<<vblocks, 256, 0, stream>>>((const uint4*)x, (uint4*)out, nvec, act);
        else
            unary_act_vec_kernel<bf16><<<vblocks, 256, 0, stream>>>((const uint4*)x, (uint4*)out, nvec, act);
        return launch_status();
    }
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == EMS_F32) unary_act_kernel<float><<<blocks, 256, 0, stream>>>((const float*)x, (float*)out, (size_t)n, act);
    else if (dtype == EMS_BF16) unary_act_kernel<bf16><<<blocks, 256, 0, stream>>>((const bf16*)x, (bf16*)out, (size_t)n, act);
    else return EMS_ERR_DTYPE;
    return launch_status();
}

EMS_EXPORT int ems_qk_prep(void* proj, long long ld, int dtype, int n, int nh, int nkv, int D, const int* positions,
                           const int* row_of_token, const float* table, int rot, int pairing, int normed, float eps,
                           void* kc, void* vc, const int* bt, int bt_stride, int page_size, int values_are_keys,
                           int write_kv, int DV, int v_normed, float v_eps, const float* v_table, int v_pairing,
                           const void* q_gain, const void* k_gain, int gain_dtype, int norm_first,
                           cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    if (DV <= 0) DV = D;
    if (D <= 0 || nh <= 0 || nkv <= 0 || rot < 0 || rot % 2 || rot > D || (rot > 0 && !table) ||
        (write_kv && (!kc || !vc || !bt || page_size <= 0)) || (values_are_keys && (DV != D || v_normed || v_table)) ||
        (v_table && DV % 2))
        return EMS_ERR_SHAPE;
    const int heads = nh + nkv + (values_are_keys ? 0 : nkv);
    int warps = heads < 8 ? heads : 8;
    const size_t smem = sizeof(float) * (size_t)warps * (D > DV ? D : DV);
    if (smem > 48 * 1024) return EMS_ERR_SHAPE;
    const float* tab = rot > 0 ? table : nullptr;
    if (dtype == EMS_F32)
        qk_prep_kernel<float><<<n, warps * 32, smem, stream>>>((float*)proj, ld, nh, nkv, D, positions, row_of_token, tab,
                                                               rot, pairing, normed, eps, (float*)kc, (float*)vc, bt,
                                                               bt_stride, page_size, values_are_keys, write_kv, DV,
                                                               v_normed, v_eps, v_table, v_pairing, q_gain, k_gain,
                                                               gain_dtype, norm_first);
    else if (dtype == EMS_BF16)
        qk_prep_kernel<bf16><<<n, warps * 32, smem, stream>>>((bf16*)proj, ld, nh, nkv, D, positions, row_of_token, tab,
                                                              rot, pairing, normed, eps, (bf16*)kc, (bf16*)vc, bt,
                                                              bt_stride, page_size, values_are_keys, write_kv, DV,
                                                              v_normed, v_eps, v_table, v_pairing, q_gain, k_gain,
                                                              gain_dtype, norm_first);
    else
        return EMS_ERR_DTYPE;
    return launch_status();
}

EMS_EXPORT int ems_norm_mean2(const void* a, const void* b, const void* wa, const void* wb, int w_dtype, void* out,
                              int dtype, int n, int C, float eps, cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    int th = 32;
    while (th < 256 && th * 4 < C) th <<= 1;
    if (dtype == EMS_F32)
        norm_mean2_kernel<float><<<n, th, 0, stream>>>((const float*)a, (const float*)b, wa, wb, w_dtype, (float*)out, C, eps);
    else if (dtype == EMS_BF16)
        norm_mean2_kernel<bf16><<<n, th, 0, stream>>>((const bf16*)a, (const bf16*)b, wa, wb, w_dtype, (bf16*)out, C, eps);
    else
        return EMS_ERR_DTYPE;
    return launch_status();
}
