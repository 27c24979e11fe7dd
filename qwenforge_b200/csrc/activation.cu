// SwiGLU gate of the feed-forward: out[t][i] = silu(gu[t][i]) * gu[t][I + i], silu(x) = x / (1 + exp(-x)),
// evaluated in float32 on the fused [gate | up] projection.
#include "common.cuh"

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / inter, c = i % inter;
        const float g = Num<T>::to_f(gu[t * 2 * inter + c]);
        const float u = Num<T>::to_f(gu[t * 2 * inter + inter + c]);
        out[i] = Num<T>::from_f(g / (1.0f + expf(-g)) * u);
    }
}

// Eight bf16 elements per thread (16-byte loads and stores); needs inter % 8 == 0 and 16-byte aligned rows.
__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int inter, size_t total8) {
    grid_chain_entry();
    const int per_row = inter / 8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / per_row, c = (i % per_row) * 8;
        const uint4 g4 = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + c);
        const uint4 u4 = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + inter + c);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
        uint4 o4;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
            o2[j] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
        }
        *reinterpret_cast<uint4*>(out + t * inter + c) = o4;
    }
}

QF_EXPORT int qf_swiglu(int is_bf16, const void* gu, void* out, int rows, int inter, cudaStream_t stream) {
    const size_t total = (size_t)rows * inter;
    if (total == 0) return 0;
    const size_t most = (size_t)(qf_sm_count() > 0 ? qf_sm_count() : 1) * 16;  // blocks that a grid-stride loop is given
    const int blocks = (int)((total + 255) / 256 < most ? (total + 255) / 256 : most);
    int code;
    if (is_bf16 && inter % 8 == 0 && ((uintptr_t)gu % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
        const size_t total8 = total / 8;
        const int b8 = (int)((total8 + 255) / 256 < most ? (total8 + 255) / 256 : most);
        code = (int)launch_pdl(swiglu_bf16x8_kernel, dim3(b8), dim3(256), 0, stream, (const bf16*)gu, (bf16*)out, inter, total8);
    } else if (is_bf16)
        code = (int)launch_pdl(swiglu_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)gu, (bf16*)out, inter, total);
    else
        code = (int)launch_pdl(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, (float*)out, inter, total);
    return code;
}

// The gate of a feed-forward with clamped halves, on the fused [gate | up] projection, in float32:
//   g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(alpha * g) * (u + 1)
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total, float limit, float alpha) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / inter, c = i % inter;
        const float g = fminf(Num<T>::to_f(gu[t * 2 * inter + c]), limit);
        const float u = fminf(fmaxf(Num<T>::to_f(gu[t * 2 * inter + inter + c]), -limit), limit);
        out[i] = Num<T>::from_f(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
    }
}

// Eight bf16 elements per thread (16-byte loads and stores); needs inter % 8 == 0 and 16-byte aligned rows.
__global__ void clamped_glu_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int inter, size_t total8, float limit,
                                          float alpha) {
    grid_chain_entry();
    const int per_row = inter / 8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / per_row, c = (i % per_row) * 8;
        const uint4 g4 = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + c);
        const uint4 u4 = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + inter + c);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
        uint4 o4;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
            g.x = fminf(g.x, limit);
            g.y = fminf(g.y, limit);
            u.x = fminf(fmaxf(u.x, -limit), limit);
            u.y = fminf(fmaxf(u.y, -limit), limit);
            o2[j] = __floats2bfloat162_rn(g.x / (1.0f + expf(-alpha * g.x)) * (u.x + 1.0f), g.y / (1.0f + expf(-alpha * g.y)) * (u.y + 1.0f));
        }
        *reinterpret_cast<uint4*>(out + t * inter + c) = o4;
    }
}

QF_EXPORT int qf_clamped_glu(int is_bf16, const void* gu, void* out, int rows, int inter, float limit, float alpha,
                             cudaStream_t stream) {
    const size_t total = (size_t)rows * inter;
    if (total == 0) return 0;
    const size_t most = (size_t)(qf_sm_count() > 0 ? qf_sm_count() : 1) * 16;
    const int blocks = (int)((total + 255) / 256 < most ? (total + 255) / 256 : most);
    if (is_bf16 && inter % 8 == 0 && ((uintptr_t)gu % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
        const size_t total8 = total / 8;
        const int b8 = (int)((total8 + 255) / 256 < most ? (total8 + 255) / 256 : most);
        return (int)launch_pdl(clamped_glu_bf16x8_kernel, dim3(b8), dim3(256), 0, stream, (const bf16*)gu, (bf16*)out, inter, total8, limit, alpha);
    }
    if (is_bf16)
        return (int)launch_pdl(clamped_glu_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)gu, (bf16*)out, inter, total, limit, alpha);
    return (int)launch_pdl(clamped_glu_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, (float*)out, inter, total, limit, alpha);
}

// SwiGLU on rows whose input was to be scaled: out[r][i] = silu(s_r * g) * (s_r * u) for the fused [gate | up] product of
// the UNSCALED rows (W (s h) = s (W h): the scale moves from the product's input to its float32 result).
template <typename T>
__global__ void scaled_swiglu_kernel(const T* __restrict__ gu, const float* __restrict__ row_scale, T* __restrict__ out, int inter,
                                     size_t total) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / inter, c = i % inter;
        const float s = row_scale[t];
        const float g = s * Num<T>::to_f(gu[t * 2 * inter + c]);
        const float u = s * Num<T>::to_f(gu[t * 2 * inter + inter + c]);
        out[i] = Num<T>::from_f(g / (1.0f + expf(-g)) * u);
    }
}

QF_EXPORT int qf_scaled_swiglu(int is_bf16, const void* gu, const float* row_scale, void* out, int rows, int inter,
                               cudaStream_t stream) {
    const size_t total = (size_t)rows * inter;
    if (total == 0) return 0;
    const size_t most = (size_t)(qf_sm_count() > 0 ? qf_sm_count() : 1) * 16;
    const int blocks = (int)((total + 255) / 256 < most ? (total + 255) / 256 : most);
    if (is_bf16)
        return (int)launch_pdl(scaled_swiglu_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)gu, row_scale, (bf16*)out, inter, total);
    return (int)launch_pdl(scaled_swiglu_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, row_scale, (float*)out, inter, total);
}

// out = act(x + bias): the first half of a feed-forward without a gate. kind 0: the square of relu, 1: tanh-GELU,
// 2: silu, 3: relu, 4: GELU in its exact form, z Phi(z) through erf, 5: tanh. Float32 inside; bias may be null.

template <typename T>
__global__ void bias_act_kernel(const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ out, int width, size_t total,
                                int kind) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const float z = Num<T>::to_f(x[i]) + (bias ? Num<T>::to_f(bias[i % width]) : 0.f);
        out[i] = Num<T>::from_f(activate(z, kind));
    }
}

// Eight bf16 elements per thread; needs width % 8 == 0 and 16-byte aligned pointers.
__global__ void bias_act_bf16x8_kernel(const bf16* __restrict__ x, const bf16* __restrict__ bias, bf16* __restrict__ out, int width,
                                       size_t total8, int kind) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 x4 = *reinterpret_cast<const uint4*>(x + i * 8);
        uint4 b4 = make_uint4(0u, 0u, 0u, 0u);
        if (bias) b4 = *reinterpret_cast<const uint4*>(bias + (i * 8) % width);
        const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&x4);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b4);
        uint4 o4;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 v = __bfloat1622float2(x2[j]), b = __bfloat1622float2(b2[j]);
            o2[j] = __floats2bfloat162_rn(activate(v.x + b.x, kind), activate(v.y + b.y, kind));
        }
        *reinterpret_cast<uint4*>(out + i * 8) = o4;
    }
}

QF_EXPORT int qf_bias_act(int is_bf16, const void* x, const void* bias, void* out, int rows, int width, int kind,
                          cudaStream_t stream) {
    const size_t total = (size_t)rows * width;
    if (total == 0) return 0;
    if (kind < 0 || kind > 5) return (int)cudaErrorInvalidValue;
    const size_t most = (size_t)(qf_sm_count() > 0 ? qf_sm_count() : 1) * 16;
    const int blocks = (int)((total + 255) / 256 < most ? (total + 255) / 256 : most);
    if (is_bf16 && width % 8 == 0 && ((uintptr_t)x | (uintptr_t)out | (uintptr_t)bias) % 16 == 0) {
        const size_t total8 = total / 8;
        const int b8 = (int)((total8 + 255) / 256 < most ? (total8 + 255) / 256 : most);
        return (int)launch_pdl(bias_act_bf16x8_kernel, dim3(b8), dim3(256), 0, stream, (const bf16*)x, (const bf16*)bias, (bf16*)out,
                               width, total8, kind);
    }
    if (is_bf16)
        return (int)launch_pdl(bias_act_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)x, (const bf16*)bias, (bf16*)out,
                               width, total, kind);
    return (int)launch_pdl(bias_act_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)x, (const float*)bias, (float*)out,
                           width, total, kind);
}

// x <- cap * tanh(x / cap) in place, float32 (logits).
__global__ void softcap_kernel(float* __restrict__ x, size_t total, float cap) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] / cap);
}

QF_EXPORT int qf_softcap(float* x, long long total, float cap, cudaStream_t stream) {
    if (total <= 0) return 0;
    const size_t most = (size_t)(qf_sm_count() > 0 ? qf_sm_count() : 1) * 16;
    const size_t want = ((size_t)total + 255) / 256;
    return (int)launch_pdl(softcap_kernel, dim3((unsigned)(want < most ? want : most)), dim3(256), 0, stream, x, (size_t)total, cap);
}

// A gate per token and head on an attention's output, in place: x[t][h][:] *= sigmoid(gate[t][h]). The gates are columns
// of a wider row (`gate_stride` elements from one token's to the next's); the sigmoid and the product are float32.
template <typename T>
__global__ void __launch_bounds__(256)
head_gate_kernel(T* __restrict__ x, const T* __restrict__ gate, int gate_stride, int n_heads, int head_dim, size_t total) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t th = i / head_dim, t = th / n_heads, h = th % n_heads;
        const float g = Num<T>::to_f(gate[t * gate_stride + h]);
        x[i] = Num<T>::from_f(Num<T>::to_f(x[i]) / (1.f + expf(-g)));
    }
}

// The same, 16 bytes of one head at a time (head_dim a multiple of what 16 bytes hold, x aligned).
template <typename T>
__global__ void __launch_bounds__(256)
head_gate_vec_kernel(T* __restrict__ x, const T* __restrict__ gate, int gate_stride, int n_heads, int head_dim, size_t groups) {
    constexpr int V = 16 / (int)sizeof(T);
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < groups; i += (size_t)gridDim.x * blockDim.x) {
        const size_t th = i * V / head_dim, t = th / n_heads, h = th % n_heads;
        const float g = Num<T>::to_f(gate[t * gate_stride + h]);
        const float s = 1.f + expf(-g);
        T v[V];
        *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(x + i * V);
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = Num<T>::from_f(Num<T>::to_f(v[j]) / s);
        *reinterpret_cast<uint4*>(x + i * V) = *reinterpret_cast<const uint4*>(v);
    }
}

QF_EXPORT int qf_head_gate(int is_bf16, void* x, const void* gate, int gate_stride, int rows, int n_heads, int head_dim,
                           cudaStream_t stream) {
    const size_t total = (size_t)rows * n_heads * head_dim;
    if (total == 0) return 0;
    const size_t most = (size_t)(qf_sm_count() > 0 ? qf_sm_count() : 1) * 16;
    const int per = is_bf16 ? 8 : 4;
    if (head_dim % per == 0 && ((uintptr_t)x & 15) == 0) {
        const size_t groups = total / per;
        const int blocks = (int)((groups + 255) / 256 < most ? (groups + 255) / 256 : most);
        if (is_bf16)
            return (int)launch_pdl(head_gate_vec_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (bf16*)x, (const bf16*)gate,
                                   gate_stride, n_heads, head_dim, groups);
        return (int)launch_pdl(head_gate_vec_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x, (const float*)gate,
                               gate_stride, n_heads, head_dim, groups);
    }
    const int blocks = (int)((total + 255) / 256 < most ? (total + 255) / 256 : most);
    if (is_bf16)
        return (int)launch_pdl(head_gate_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (bf16*)x, (const bf16*)gate, gate_stride,
                               n_heads, head_dim, total);
    return (int)launch_pdl(head_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x, (const float*)gate, gate_stride,
                           n_heads, head_dim, total);
}

// A gated feed-forward's middle with any of the activations above and optional biases: from the fused [gate | up] product,
//   out[t][i] = act(gate[t][i] + bias[i]) * (up[t][i] + bias[inter + i]),  float32 inside.
template <typename T>
__global__ void __launch_bounds__(256)
bias_glu_kernel(const T* __restrict__ gu, const T* __restrict__ bias, T* __restrict__ out, int inter, size_t total, int kind) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / inter, c = i % inter;
        float g = Num<T>::to_f(gu[t * 2 * inter + c]), u = Num<T>::to_f(gu[t * 2 * inter + inter + c]);
        if (bias) {
            g += Num<T>::to_f(bias[c]);
            u += Num<T>::to_f(bias[inter + c]);
        }
        out[i] = Num<T>::from_f(activate(g, kind) * u);
    }
}

// Eight bf16 elements per thread; needs inter % 8 == 0 and 16-byte aligned pointers.
__global__ void __launch_bounds__(256)
bias_glu_bf16x8_kernel(const bf16* __restrict__ gu, const bf16* __restrict__ bias, bf16* __restrict__ out, int inter, size_t total8,
                       int kind) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i * 8 / inter, c = i * 8 % inter;
        const uint4 g4 = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + c);
        const uint4 u4 = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + inter + c);
        uint4 bg4 = make_uint4(0u, 0u, 0u, 0u), bu4 = bg4;
        if (bias) {
            bg4 = *reinterpret_cast<const uint4*>(bias + c);
            bu4 = *reinterpret_cast<const uint4*>(bias + inter + c);
        }
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
        const __nv_bfloat162* bg2 = reinterpret_cast<const __nv_bfloat162*>(&bg4);
        const __nv_bfloat162* bu2 = reinterpret_cast<const __nv_bfloat162*>(&bu4);
        uint4 o4;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
            const float2 bg = __bfloat1622float2(bg2[j]), bu = __bfloat1622float2(bu2[j]);
            o2[j] = __floats2bfloat162_rn(activate(g.x + bg.x, kind) * (u.x + bu.x), activate(g.y + bg.y, kind) * (u.y + bu.y));
        }
        *reinterpret_cast<uint4*>(out + i * 8) = o4;
    }
}

QF_EXPORT int qf_bias_glu(int is_bf16, const void* gu, const void* bias, void* out, int rows, int inter, int kind,
                          cudaStream_t stream) {
    const size_t total = (size_t)rows * inter;
    if (total == 0) return 0;
    if (kind < 0 || kind > 5) return (int)cudaErrorInvalidValue;
    const size_t most = (size_t)(qf_sm_count() > 0 ? qf_sm_count() : 1) * 16;
    if (is_bf16 && inter % 8 == 0 && ((uintptr_t)gu | (uintptr_t)out | (uintptr_t)bias) % 16 == 0) {
        const size_t total8 = total / 8;
        const int b8 = (int)((total8 + 255) / 256 < most ? (total8 + 255) / 256 : most);
        return (int)launch_pdl(bias_glu_bf16x8_kernel, dim3(b8), dim3(256), 0, stream, (const bf16*)gu, (const bf16*)bias, (bf16*)out,
                               inter, total8, kind);
    }
    const int blocks = (int)((total + 255) / 256 < most ? (total + 255) / 256 : most);
    if (is_bf16)
        return (int)launch_pdl(bias_glu_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)gu, (const bf16*)bias, (bf16*)out,
                               inter, total, kind);
    return (int)launch_pdl(bias_glu_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, (const float*)bias, (float*)out,
                           inter, total, kind);
}
