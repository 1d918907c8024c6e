// Row-wise kernels around the residual stream for decoders with a norm on both sides of every
// sub-layer: a vector added to the stream between layers, the grouped RMSNorm fused with the
// norm of the delta that joins the stream before it, gated activations other than SiLU, and
// the short causal convolution over time with its per-request state.
//
// All arithmetic is 32-bit; the storage type T is float (the true 32-bit path) or bfloat16.
//
//   grouped RMSNorm   the vector is cut into G equal consecutive parts; part g is divided by
//                     sqrt(mean(part^2) + eps); the whole is multiplied by the gain.  Nothing
//                     is rounded between the division and the gain.
//   post + pre norm   residual += norm_post(delta);  out = norm_pre(residual)
//   causal taps       out[t] = h[t] + sum_j w[:, j] * h[t - taps + 1 + j], h = 0 before the
//                     request's first token; the last taps - 1 inputs of a request are its state
#include "common.cuh"

namespace ems {

// ---------------------------------------------------------------------------------------
// residual[n, :] += embed[tokens[n], :] + table[row, :]   (either may be absent)

template <typename T>
__global__ void stream_inject_kernel(float* __restrict__ residual, const int* __restrict__ tokens,
                                     const int* __restrict__ deferred, const T* __restrict__ embed,
                                     const T* __restrict__ vec, int H) {
    const size_t n = blockIdx.x;
    const T* e = nullptr;
    if (embed) {
        int tok = tokens[n];
        if (tok < 0) tok = deferred ? deferred[-(tok + 1)] : 0;
        e = embed + (size_t)tok * H;
    }
    float* r = residual + n * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float s = r[i];
        if (e) s += to_f32<T>(e[i]);
        if (vec) s += to_f32<T>(vec[i]);
        r[i] = s;
    }
}

// ---------------------------------------------------------------------------------------
// One block per output row.  buf (dynamic shared memory) holds the row in 32 bits between the
// phases, followed by one factor per group.  The order of every sum depends on blockDim and the
// sizes only.

template <typename T>
__global__ void add_norm_grouped_kernel(const T* __restrict__ delta, const void* __restrict__ post_gain,
                                        int pg_dtype, int post_groups, float post_eps, float* residual,
                                        const void* __restrict__ gain, int g_dtype, int groups, float eps,
                                        T* __restrict__ out, const int* __restrict__ rows, int H,
                                        int write_residual) {
    extern __shared__ float buf[];
    __shared__ float red[33];
    float* stat = buf + H;
    const size_t r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : r;
    float* res = residual + src * H;
    const T* dl = delta ? delta + src * H : nullptr;
    if (dl && post_gain) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) buf[i] = to_f32<T>(dl[i]);
        __syncthreads();
        const int gs = H / post_groups;
        for (int g = 0; g < post_groups; ++g) {
            float ss = 0.f;
            for (int i = threadIdx.x; i < gs; i += blockDim.x) {
                const float v = buf[g * gs + i];
                ss += v * v;
            }
            const float total = block_sum(ss, red);
            if (threadIdx.x == 0) stat[g] = 1.0f / sqrtf(total / (float)gs + post_eps);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float s = res[i] + buf[i] * stat[i / gs] * load_any(post_gain, pg_dtype, i);
            buf[i] = s;
            if (write_residual) res[i] = s;
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float s = res[i];
            if (dl) {
                s += to_f32<T>(dl[i]);
                if (write_residual) res[i] = s;
            }
            buf[i] = s;
        }
    }
    __syncthreads();
    const int gs = H / groups;
    for (int g = 0; g < groups; ++g) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < gs; i += blockDim.x) {
            const float v = buf[g * gs + i];
            ss += v * v;
        }
        const float total = block_sum(ss, red);  // (its barriers also order the reads of stat above)
        if (threadIdx.x == 0) stat[g] = 1.0f / sqrtf(total / (float)gs + eps);
    }
    __syncthreads();
    T* o = out + r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        o[i] = from_f32<T>(buf[i] * stat[i / gs] * load_any(gain, g_dtype, i));
}


// The same with four columns per thread held in registers between the phases (H and the group
// sizes multiples of 4, H <= 4 * VPT * blockDim): a row is one round trip to memory.
template <typename T> struct Vec4s;
template <> struct Vec4s<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec4s<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[4]) {
        const uint2 t = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[4]) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 t;
        t.x = *reinterpret_cast<const uint32_t*>(&a);
        t.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = t;
    }
};

__device__ __forceinline__ void load_gain4(const void* w, int dtype, int col, float (&v)[4]) {
    if (dtype == EMS_F32) Vec4s<float>::load(reinterpret_cast<const float*>(w) + col, v);
    else Vec4s<bf16>::load(reinterpret_cast<const bf16*>(w) + col, v);
}

// Per-group factors 1 / sqrt(mean + eps) from each thread's share `ss[v]` of the sum of squares of
// its chunk v (whose group is grp[v]); left in stat[0 .. groups).
template <int VPT>
__device__ __forceinline__ void group_factors(const float (&ss)[VPT], const int (&grp)[VPT], int groups, int gs,
                                              float eps, float* stat, float* red) {
    for (int g = 0; g < groups; ++g) {
        float mine = 0.f;
#pragma unroll
        for (int v = 0; v < VPT; ++v)
            if (grp[v] == g) mine += ss[v];
        const float total = block_sum(mine, red);
        if (threadIdx.x == 0) stat[g] = 1.0f / sqrtf(total / (float)gs + eps);
    }
    __syncthreads();
}

template <typename T, int VPT>
__global__ void add_norm_grouped_vec_kernel(const T* __restrict__ delta, const void* __restrict__ post_gain,
                                            int pg_dtype, int post_groups, float post_eps, float* residual,
                                            const void* __restrict__ gain, int g_dtype, int groups, float eps,
                                            T* __restrict__ out, const int* __restrict__ rows, int H,
                                            int write_residual) {
    __shared__ float red[33];
    __shared__ float stat[64], stat2[64];
    const size_t r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : r;
    float* res = residual + src * H;
    const T* dl = delta ? delta + src * H : nullptr;
    float x[VPT][4], ss[VPT];
    int grp[VPT];
    const int gs_post = post_gain ? H / post_groups : H, gs = H / groups;
    if (dl && post_gain) {
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int col = (v * blockDim.x + threadIdx.x) * 4;
            ss[v] = 0.f;
            grp[v] = -1;
            if (col < H) {
                Vec4s<T>::load(dl + col, x[v]);
                grp[v] = col / gs_post;
#pragma unroll
                for (int i = 0; i < 4; ++i) ss[v] += x[v][i] * x[v][i];
            }
        }
        group_factors<VPT>(ss, grp, post_groups, gs_post, post_eps, stat, red);
    }
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int col = (v * blockDim.x + threadIdx.x) * 4;
        ss[v] = 0.f;
        if (col < H) {
            float rr[4];
            Vec4s<float>::load(res + col, rr);
            if (dl && post_gain) {
                float w[4];
                load_gain4(post_gain, pg_dtype, col, w);
                const float f = stat[grp[v]];
#pragma unroll
                for (int i = 0; i < 4; ++i) rr[i] += x[v][i] * f * w[i];
            } else if (dl) {
                float d[4];
                Vec4s<T>::load(dl + col, d);
#pragma unroll
                for (int i = 0; i < 4; ++i) rr[i] += d[i];
            }
            if (dl && write_residual) Vec4s<float>::store(res + col, rr);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                x[v][i] = rr[i];
                ss[v] += rr[i] * rr[i];
            }
            grp[v] = col / gs;
        } else {
            grp[v] = -1;
        }
    }
    group_factors<VPT>(ss, grp, groups, gs, eps, stat2, red);
    T* o = out + r * H;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int col = (v * blockDim.x + threadIdx.x) * 4;
        if (col < H) {
            float w[4], y[4];
            load_gain4(gain, g_dtype, col, w);
            const float f = stat2[grp[v]];
#pragma unroll
            for (int i = 0; i < 4; ++i) y[i] = x[v][i] * f * w[i];
            Vec4s<T>::store(o + col, y);
        }
    }
}

// ---------------------------------------------------------------------------------------
// out[n, i] = act(gu[n, i]) * gu[n, I + i];  act: 0 SiLU, 1 ReLU, 2 GELU (tanh form); 3 the capped form:
// with g = min(gate, limit) and u = clamp(up, -limit, limit) it is g * sigmoid(alpha * g) * (u + 1).
// A row of gu has `ld` elements; with row_gate, column 2 I of the row holds a number z and the whole
// output row is multiplied by sigmoid(z).

__device__ __forceinline__ float glu_activation(float g, int act) {
    if (act == 1) return fmaxf(g, 0.f);
    if (act == 2) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return g / (1.f + expf(-g));
}

template <typename T>
__global__ void glu_act_kernel(const T* __restrict__ gu, long long ld, T* __restrict__ out, int I, int act,
                               float limit, float alpha, int row_gate) {
    const size_t n = blockIdx.x;
    const T* g = gu + n * ld;
    T* o = out + n * I;
    const float rg = row_gate ? 1.f / (1.f + expf(-to_f32<T>(g[2 * I]))) : 1.f;
    for (int i = threadIdx.x; i < I; i += blockDim.x) {
        float gv = to_f32<T>(g[i]), uv = to_f32<T>(g[I + i]), y;
        if (act == 3) {
            gv = fminf(gv, limit);
            uv = fminf(fmaxf(uv, -limit), limit);
            y = gv / (1.f + expf(-alpha * gv)) * (uv + 1.f);
        } else {
            y = glu_activation(gv, act) * uv;
        }
        o[i] = from_f32<T>(y * rg);
    }
}

// ---------------------------------------------------------------------------------------
// causal taps.  x: [N, C] packed rows; w: [C, taps]; state: [slots, taps - 1, C] float, the last
// taps - 1 inputs of each request in time order (zero where the request has not begun).

template <typename T>
__global__ void causal_taps_kernel(const T* __restrict__ x, long long ldx, const void* __restrict__ w, int w_dtype,
                                   const void* __restrict__ bias, int identity,
                                   const float* __restrict__ state, const int* __restrict__ slots,
                                   const int* __restrict__ cu_q, const int* __restrict__ row_of_token,
                                   T* __restrict__ out, int C, int taps) {
    const int t = blockIdx.x;
    const int row = row_of_token[t];
    const int first = cu_q[row];
    const int local = t - first;
    const float* st = state ? state + (size_t)slots[row] * (taps - 1) * C : nullptr;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float conv = bias ? load_any(bias, w_dtype, c) : 0.f;
        for (int j = 0; j < taps; ++j) {
            const int s = local - (taps - 1) + j;
            float v;
            if (s >= 0) v = to_f32<T>(x[(size_t)(first + s) * ldx + c]);
            else v = st ? st[(size_t)(taps - 1 + s) * C + c] : 0.f;
            conv += load_any(w, w_dtype, (size_t)c * taps + j) * v;
        }
        out[(size_t)t * C + c] = from_f32<T>(identity ? to_f32<T>(x[(size_t)t * ldx + c]) + conv : conv);
    }
}

// After the convolution has read the old state: the last taps - 1 inputs of every row, from the
// step's tokens and, where the row brought fewer, from the old state moved up.  A thread owns a
// channel, reads entries above the one it writes, and so needs no second buffer.
template <typename T>
__global__ void causal_taps_state_kernel(const T* __restrict__ x, long long ldx, float* __restrict__ state,
                                         const int* __restrict__ slots, const int* __restrict__ cu_q, int C,
                                         int taps) {
    const int row = blockIdx.x;
    const int first = cu_q[row], q = cu_q[row + 1] - first;
    if (q <= 0) return;
    float* st = state + (size_t)slots[row] * (taps - 1) * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        for (int s = 0; s < taps - 1; ++s) {
            const int src = q - (taps - 1) + s;
            st[(size_t)s * C + c] = src >= 0 ? to_f32<T>(x[(size_t)(first + src) * ldx + c])
                                             : st[(size_t)(s + q) * C + c];
        }
    }
}

// A step in which every row brings one token: convolution and state in one kernel.  A thread owns
// (row, channel), reads the state it then rewrites.
template <typename T>
__global__ void causal_taps_single_kernel(const T* __restrict__ x, long long ldx, const void* __restrict__ w,
                                          int w_dtype, const void* __restrict__ bias, int identity,
                                          float* __restrict__ state, const int* __restrict__ slots,
                                          T* __restrict__ out, int C, int taps) {
    const int row = blockIdx.x;
    float* st = state + (size_t)slots[row] * (taps - 1) * C;
    // (blocks along y share a row's channels, so that a wide row is not one block's loop)
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        const float h = to_f32<T>(x[(size_t)row * ldx + c]);
        float conv = bias ? load_any(bias, w_dtype, c) : 0.f;
        for (int j = 0; j < taps - 1; ++j) {
            const float v = st[(size_t)j * C + c];
            conv += load_any(w, w_dtype, (size_t)c * taps + j) * v;
            if (j > 0) st[(size_t)(j - 1) * C + c] = v;
        }
        conv += load_any(w, w_dtype, (size_t)c * taps + taps - 1) * h;
        st[(size_t)(taps - 2) * C + c] = h;
        out[(size_t)row * C + c] = from_f32<T>(identity ? h + conv : conv);
    }
}

static int threads_for(int n) {
    int t = 32;
    while (t < n && t < 256) t <<= 1;
    return t;
}

}  // namespace ems

using namespace ems;

EMS_EXPORT int ems_stream_inject(void* residual, const int* tokens, const int* deferred, const void* embed,
                                 const void* vec, int dtype, int n, int H, cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    const int th = threads_for(H);
    if (dtype == EMS_F32)
        stream_inject_kernel<float><<<n, th, 0, stream>>>((float*)residual, tokens, deferred, (const float*)embed,
                                                          (const float*)vec, H);
    else if (dtype == EMS_BF16)
        stream_inject_kernel<bf16><<<n, th, 0, stream>>>((float*)residual, tokens, deferred, (const bf16*)embed,
                                                         (const bf16*)vec, H);
    else
        return EMS_ERR_DTYPE;
    return launch_status();
}

EMS_EXPORT int ems_add_norm_grouped(const void* delta, const void* post_gain, int pg_dtype, int post_groups,
                                    float post_eps, void* residual, const void* gain, int g_dtype, int groups,
                                    float eps, void* out, int dtype, const int* rows, int n, int H,
                                    int write_residual, cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    if (groups <= 0 || H % groups || (post_gain && (post_groups <= 0 || H % post_groups))) return EMS_ERR_SHAPE;
    const int most = groups > post_groups ? groups : post_groups;
    // four columns per thread in registers where the sizes allow: one trip to memory per row
    const bool aligned = !(reinterpret_cast<uintptr_t>(delta) & 15) && !(reinterpret_cast<uintptr_t>(residual) & 15) &&
                         !(reinterpret_cast<uintptr_t>(out) & 15) && !(reinterpret_cast<uintptr_t>(gain) & 15) &&
                         !(reinterpret_cast<uintptr_t>(post_gain) & 15);
    if (aligned && H % 4 == 0 && (H / groups) % 4 == 0 && (!post_gain || (H / post_groups) % 4 == 0) && most <= 64 &&
        H <= 4 * 8 * 256) {
        int th = 32;
        while (th < 256 && th * 4 < H) th <<= 1;
        const int vpt = (H + 4 * th - 1) / (4 * th);
#define EMS_LAUNCH_NORM_VEC(T, V)                                                                              \
    add_norm_grouped_vec_kernel<T, V><<<n, th, 0, stream>>>((const T*)delta, post_gain, pg_dtype, post_groups, \
                                                            post_eps, (float*)residual, gain, g_dtype, groups, \
                                                            eps, (T*)out, rows, H, write_residual)
#define EMS_NORM_VEC_BY_VPT(T)                         \
    do {                                               \
        if (vpt <= 1) EMS_LAUNCH_NORM_VEC(T, 1);       \
        else if (vpt <= 2) EMS_LAUNCH_NORM_VEC(T, 2);  \
        else if (vpt <= 4) EMS_LAUNCH_NORM_VEC(T, 4);  \
        else EMS_LAUNCH_NORM_VEC(T, 8);                \
    } while (0)
        if (dtype == EMS_F32) EMS_NORM_VEC_BY_VPT(float);
        else if (dtype == EMS_BF16) EMS_NORM_VEC_BY_VPT(bf16);
        else return EMS_ERR_DTYPE;
#undef EMS_NORM_VEC_BY_VPT
#undef EMS_LAUNCH_NORM_VEC
        return launch_status();
    }
    const size_t smem = (size_t)(H + most) * sizeof(float);
    if (smem > 200 * 1024) return EMS_ERR_SHAPE;
    const int th = threads_for(H);
#define EMS_LAUNCH_NORM(T)                                                                                     \
    do {                                                                                                       \
        if (smem > 48 * 1024)                                                                                  \
            cudaFuncSetAttribute(add_norm_grouped_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                 (int)smem);                                                                   \
        add_norm_grouped_kernel<T><<<n, th, smem, stream>>>((const T*)delta, post_gain, pg_dtype, post_groups, \
                                                            post_eps, (float*)residual, gain, g_dtype, groups, \
                                                            eps, (T*)out, rows, H, write_residual);            \
    } while (0)
    if (dtype == EMS_F32) EMS_LAUNCH_NORM(float);
    else if (dtype == EMS_BF16) EMS_LAUNCH_NORM(bf16);
    else return EMS_ERR_DTYPE;
#undef EMS_LAUNCH_NORM
    return launch_status();
}

EMS_EXPORT int ems_glu_act(const void* gu, long long ld, void* out, int dtype, int n, int I, int act, float limit,
                           float alpha, int row_gate, cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    if (act < 0 || act > 3 || ld < 2 * I + (row_gate ? 1 : 0)) return EMS_ERR_SHAPE;
    const int th = threads_for(I);
    if (dtype == EMS_F32)
        glu_act_kernel<float><<<n, th, 0, stream>>>((const float*)gu, ld, (float*)out, I, act, limit, alpha, row_gate);
    else if (dtype == EMS_BF16)
        glu_act_kernel<bf16><<<n, th, 0, stream>>>((const bf16*)gu, ld, (bf16*)out, I, act, limit, alpha, row_gate);
    else return EMS_ERR_DTYPE;
    return launch_status();
}

EMS_EXPORT int ems_causal_taps(const void* x, long long ldx, const void* w, int w_dtype, const void* bias,
                               int identity, void* state, const int* slots,
                               const int* cu_q, const int* row_of_token, void* out, int dtype, int n, int rows,
                               int C, int taps, cudaStream_t stream) {
    if (n <= 0) return EMS_OK;
    if (taps < 1 || (taps > 1 && !state) || ldx < C) return EMS_ERR_SHAPE;
    const int th = threads_for(C);
#define EMS_LAUNCH_TAPS(T)                                                                                   \
    do {                                                                                                     \
        if (n == rows && taps > 1) {                                                                         \
            causal_taps_single_kernel<T><<<dim3(rows, (C + th - 1) / th), th, 0, stream>>>(                  \
                                                                  (const T*)x, ldx, w, w_dtype, bias,        \
                                                                  identity, (float*)state,                   \
                                                                  slots, (T*)out, C, taps);                  \
            break;                                                                                           \
        }                                                                                                    \
        causal_taps_kernel<T><<<n, th, 0, stream>>>((const T*)x, ldx, w, w_dtype, bias, identity,            \
                                                    (const float*)state, slots,                             \
                                                    cu_q, row_of_token, (T*)out, C, taps);                  \
        if (taps > 1)                                                                                        \
            causal_taps_state_kernel<T><<<rows, th, 0, stream>>>((const T*)x, ldx, (float*)state, slots,     \
                                                                 cu_q, C, taps);                             \
    } while (0)
    if (dtype == EMS_F32) EMS_LAUNCH_TAPS(float);
    else if (dtype == EMS_BF16) EMS_LAUNCH_TAPS(bf16);
    else return EMS_ERR_DTYPE;
#undef EMS_LAUNCH_TAPS
    return launch_status();
}
