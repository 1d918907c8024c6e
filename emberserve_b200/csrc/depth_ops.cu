// Row-wise kernels for what a decoder may do to its residual stream between layers:
//
//  * ems_add_cast: residual += delta (32-bit); xb = residual in the activation type, for a product that
//    reads the stream itself rather than a norm of it;
//  * ems_token_gate: g[n, :] = gelu_tanh(z[n, :]) * table[token(n), col0 : col0 + C], the gate of a
//    layer's own input from a second embedding table (one column range per layer);
//  * ems_depth_mix: the weighted sum over the stream's states at all depths so far.  hist holds the
//    states [depths, N, H] in 32 bits; the kernel completes the newest one (residual, plus an optional
//    delta that may first pass a unit-RMS norm with a gain), stores it as hist[count - 1] and leaves
//    sum_j w[j] * hist[j], j < count, in the residual.
//
// All sums are 32-bit and are taken in index order; the storage type T of activations is float or bfloat16.
#include "common.cuh"

namespace ems {

template <typename T>
__global__ void add_cast_kernel(const T* __restrict__ delta, float* __restrict__ residual, T* __restrict__ xb, int H) {
    const size_t n = blockIdx.x;
    float* r = residual + n * H;
    const T* d = delta ? delta + n * H : nullptr;
    T* o = xb + n * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float s = r[i];
        if (d) {
            s += to_f32<T>(d[i]);
            r[i] = s;
        }
        o[i] = from_f32<T>(s);
    }
}

template <typename T>
__global__ void token_gate_kernel(const T* __restrict__ z, const void* __restrict__ table, int t_dtype, long long ldt,
                                  int col0, const int* __restrict__ tokens, const int* __restrict__ deferred,
                                  T* __restrict__ out, int C) {
    const size_t n = blockIdx.x;
    int tok = tokens[n];
    if (tok < 0) tok = deferred ? deferred[-(tok + 1)] : 0;
    for (int i = threadIdx.x; i < C; i += blockDim.x) {
        const float v = to_f32<T>(z[n * C + i]);
        const float g = 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
        out[n * C + i] = from_f32<T>(g * load_any(table, t_dtype, (size_t)tok * ldt + col0 + i));
    }
}

template <typename T> __device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <> __device__ __forceinline__ void load4<bf16>(const bf16* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
    v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
}

// VEC4: H and the plane are multiples of 4 and every pointer is aligned for four elements
template <typename T, bool VEC4>
__global__ void depth_mix_kernel(const T* __restrict__ delta, const void* __restrict__ gain, int g_dtype, float eps,
                                 float* __restrict__ residual, float* __restrict__ hist, const float* __restrict__ w,
                                 int count, size_t plane, int H) {
    __shared__ float red[33];
    const size_t n = blockIdx.x;
    float* r = residual + n * H;
    const T* d = delta ? delta + n * H : nullptr;
    float f = 1.f;
    if (d && gain) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = to_f32<T>(d[i]);
            ss = fmaf(v, v, ss);
        }
        f = 1.0f / sqrtf(block_sum(ss, red) / (float)H + eps);
    }
    float* newest = hist + (size_t)(count - 1) * plane + n * H;
    if (VEC4) {
        // four columns per thread, the earlier states' loads of a column group in flight together; the
        // sums run over the depths in index order as in the scalar form below
        const float* hrow = hist + n * H;
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float4 x = *reinterpret_cast<const float4*>(r + i);
            if (d) {
                float dv[4];
                load4<T>(d + i, dv);
                if (gain) {
                    x.x += dv[0] * f * load_any(gain, g_dtype, i);
                    x.y += dv[1] * f * load_any(gain, g_dtype, i + 1);
                    x.z += dv[2] * f * load_any(gain, g_dtype, i + 2);
                    x.w += dv[3] * f * load_any(gain, g_dtype, i + 3);
                } else {
                    x.x += dv[0]; x.y += dv[1]; x.z += dv[2]; x.w += dv[3];
                }
            }
            *reinterpret_cast<float4*>(newest + i) = x;
            if (w) {
                float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
                for (int j = 0; j + 1 < count; ++j) {
                    const float4 h = *reinterpret_cast<const float4*>(hrow + (size_t)j * plane + i);
                    const float wj = w[j];
                    s.x = fmaf(wj, h.x, s.x); s.y = fmaf(wj, h.y, s.y); s.z = fmaf(wj, h.z, s.z); s.w = fmaf(wj, h.w, s.w);
                }
                const float wl = w[count - 1];
                x.x = fmaf(wl, x.x, s.x); x.y = fmaf(wl, x.y, s.y); x.z = fmaf(wl, x.z, s.z); x.w = fmaf(wl, x.w, s.w);
            }
            *reinterpret_cast<float4*>(r + i) = x;
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float x = r[i];
        if (d) x += gain ? to_f32<T>(d[i]) * f * load_any(gain, g_dtype, i) : to_f32<T>(d[i]);
        newest[i] = x;
        if (w) {
            float s = 0.f;
            for (int j = 0; j + 1 < count; ++j) s = fmaf(w[j], hist[(size_t)j * plane + n * H + i], s);
            x = fmaf(w[count - 1], x, s);
        }
        r[i] = x;
    }
}

static int depth_threads(int n) {
    int th = 32;
    while (th < 256 && th * 4 < n) th <<= 1;
    return th;
}

}  // namespace ems

using namespace ems;

EMS_EXPORT int ems_add_cast(const void* delta, float* residual, void* xb, int dtype, int n, int H, cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    const int th = depth_threads(H);
    if (dtype == EMS_F32) add_cast_kernel<float><<<n, th, 0, stream>>>((const float*)delta, residual, (float*)xb, H);
    else if (dtype == EMS_BF16) add_cast_kernel<bf16><<<n, th, 0, stream>>>((const bf16*)delta, residual, (bf16*)xb, H);
    else return EMS_ERR_DTYPE;
    return launch_status();
}

EMS_EXPORT int ems_token_gate(const void* z, const void* table, int t_dtype, long long ldt, int col0, const int* tokens,
                              const int* deferred, void* out, int dtype, int n, int C, cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    if (C <= 0 || col0 < 0 || col0 + C > ldt) return EMS_ERR_SHAPE;
    const int th = depth_threads(C);
    if (dtype == EMS_F32)
        token_gate_kernel<float><<<n, th, 0, stream>>>((const float*)z, table, t_dtype, ldt, col0, tokens, deferred,
                                                       (float*)out, C);
    else if (dtype == EMS_BF16)
        token_gate_kernel<bf16><<<n, th, 0, stream>>>((const bf16*)z, table, t_dtype, ldt, col0, tokens, deferred,
                                                      (bf16*)out, C);
    else return EMS_ERR_DTYPE;
    return launch_status();
}

// w may be null: the newest state is completed and stored, and stays the residual (no sum).
EMS_EXPORT int ems_depth_mix(const void* delta, const void* gain, int g_dtype, float eps, float* residual, float* hist,
                             const float* w, int count, long long plane, int dtype, int n, int H, cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    if (count < 1 || plane < (long long)n * H) return EMS_ERR_SHAPE;
    const bool vec = H % 4 == 0 && plane % 4 == 0 && ((uintptr_t)residual % 16) == 0 && ((uintptr_t)hist % 16) == 0 &&
                     ((uintptr_t)delta % 16) == 0;
    const int th = depth_threads(vec ? H / 4 : H);
    if (dtype == EMS_F32) {
        auto k = vec ? depth_mix_kernel<float, true> : depth_mix_kernel<float, false>;
        k<<<n, th, 0, stream>>>((const float*)delta, gain, g_dtype, eps, residual, hist, w, count, (size_t)plane, H);
    } else if (dtype == EMS_BF16) {
        auto k = vec ? depth_mix_kernel<bf16, true> : depth_mix_kernel<bf16, false>;
        k<<<n, th, 0, stream>>>((const bf16*)delta, gain, g_dtype, eps, residual, hist, w, count, (size_t)plane, H);
    }
    else return EMS_ERR_DTYPE;
    return launch_status();
}
