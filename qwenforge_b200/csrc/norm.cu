// RMSNorm over the float32 residual stream, fused with the residual addition that precedes it:
//   hidden += delta (if delta is given);  out = hidden * rsqrt(mean(hidden^2) + eps) * weight
// The sum of squares, the reciprocal root and the scaling are float32; `out` has the activation type.
#include "common.cuh"

template <typename T>
__global__ void add_rms_norm_kernel(float* __restrict__ hidden, const T* __restrict__ delta,
                                    const T* __restrict__ weight, T* __restrict__ out, int width, float eps) {
    grid_chain_entry();
    __shared__ float scratch[33];
    float* h = hidden + (size_t)blockIdx.x * width;
    const T* d = delta ? delta + (size_t)blockIdx.x * width : nullptr;
    T* o = out + (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = h[c];
        if (d) {
            v += Num<T>::to_f(d[c]);
            h[c] = v;
        }
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
    // each thread re-reads the columns it wrote itself
    for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = Num<T>::from_f(h[c] * inv * Num<T>::to_f(weight[c]));
}

// The same with 16-byte accesses and the row kept in registers between the two passes: width % 4 == 0 and
// width <= 4 * 4 * blockDim (4096 at 256 threads).
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 r = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        uint2 r;
        *reinterpret_cast<__nv_bfloat162*>(&r.x) = __floats2bfloat162_rn(v.x, v.y);
        *reinterpret_cast<__nv_bfloat162*>(&r.y) = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2*>(p) = r;
    }
};

template <typename T>
__global__ void __launch_bounds__(256)
add_rms_norm_vec_kernel(float* __restrict__ hidden, const T* __restrict__ delta, const T* __restrict__ weight,
                        T* __restrict__ out, int width, float eps) {
    grid_chain_entry();
    __shared__ float scratch[33];
    float* h = hidden + (size_t)blockIdx.x * width;
    const T* d = delta ? delta + (size_t)blockIdx.x * width : nullptr;
    T* o = out + (size_t)blockIdx.x * width;
    const int n4 = width / 4;
    float4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int c = threadIdx.x + u * 256;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < n4) {
            v[u] = Vec4<float>::load(h + 4 * c);
            if (d) {
                const float4 dv = Vec4<T>::load(d + 4 * c);
                v[u].x += dv.x;
                v[u].y += dv.y;
                v[u].z += dv.z;
                v[u].w += dv.w;
                Vec4<float>::store(h + 4 * c, v[u]);
            }
            ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int c = threadIdx.x + u * 256;
        if (c < n4) {
            const float4 w = Vec4<T>::load(weight + 4 * c);
            Vec4<T>::store(o + 4 * c, make_float4(v[u].x * inv * w.x, v[u].y * inv * w.y, v[u].z * inv * w.z, v[u].w * inv * w.w));
        }
    }
}

// Narrow rows (width <= 1024, a multiple of 4): a warp per row, eight rows per block. The row stays in the lanes'
// registers, the sum of squares needs shuffles only, and a lane has up to eight independent 16-byte loads in flight, where
// a block per row had one load per thread and two block-wide barriers. Which kernel runs depends on the width alone, so a
// row's result does not depend on how many rows the step has.
#define NW_ROWS 8
#define NW_MAX 8   // 16-byte groups per lane
template <typename T>
__global__ void __launch_bounds__(NW_ROWS * 32)
add_rms_norm_warp_kernel(float* __restrict__ hidden, const T* __restrict__ delta, const T* __restrict__ weight,
                         T* __restrict__ out, int rows, int width, float eps) {
    grid_chain_entry();
    const int row = blockIdx.x * NW_ROWS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    float* h = hidden + (size_t)row * width;
    const T* d = delta ? delta + (size_t)row * width : nullptr;
    T* o = out + (size_t)row * width;
    const int n4 = width / 4;
    float4 v[NW_MAX], dv[NW_MAX];
#pragma unroll
    for (int u = 0; u < NW_MAX; ++u) {
        const int c = lane + 32 * u;
        v[u] = c < n4 ? Vec4<float>::load(h + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
        dv[u] = (d && c < n4) ? Vec4<T>::load(d + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < NW_MAX; ++u) {
        const int c = lane + 32 * u;
        if (d && c < n4) {
            v[u].x += dv[u].x;
            v[u].y += dv[u].y;
            v[u].z += dv[u].z;
            v[u].w += dv[u].w;
            Vec4<float>::store(h + 4 * c, v[u]);
        }
        ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)width + eps);
#pragma unroll
    for (int u = 0; u < NW_MAX; ++u) {
        const int c = lane + 32 * u;
        if (c < n4) {
            const float4 w = Vec4<T>::load(weight + 4 * c);
            Vec4<T>::store(o + 4 * c, make_float4(v[u].x * inv * w.x, v[u].y * inv * w.y, v[u].z * inv * w.z, v[u].w * inv * w.w));
        }
    }
}

template <typename T>
static int launch(float* hidden, const void* delta, const void* weight, void* out, int rows, int width, float eps,
                  cudaStream_t stream) {
    if (rows <= 0) return 0;
    const uintptr_t align = (uintptr_t)hidden | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out;
    if (width % 4 == 0 && width <= 4 * 32 * NW_MAX && align % 16 == 0) {
        return (int)launch_pdl(add_rms_norm_warp_kernel<T>, dim3((rows + NW_ROWS - 1) / NW_ROWS), dim3(NW_ROWS * 32), 0, stream, hidden, (const T*)delta, (const T*)weight,
                                                                                              (T*)out, rows, width, eps);
    }
    if (width % 4 == 0 && width <= 4096 && align % 16 == 0) {
        return (int)launch_pdl(add_rms_norm_vec_kernel<T>, dim3(rows), dim3(256), 0, stream, hidden, (const T*)delta, (const T*)weight, (T*)out, width, eps);
    }
    return (int)launch_pdl(add_rms_norm_kernel<T>, dim3(rows), dim3(256), 0, stream, hidden, (const T*)delta, (const T*)weight, (T*)out, width, eps);
}

QF_EXPORT int qf_add_rms_norm(int is_bf16, float* hidden, const void* delta, const void* weight, void* out, int rows,
                              int width, float eps, cudaStream_t stream) {
    return is_bf16 ? launch<bf16>(hidden, delta, weight, out, rows, width, eps, stream)
                   : launch<float>(hidden, delta, weight, out, rows, width, eps, stream);
}

template <typename T> __global__ void residual_add_kernel(float* __restrict__ hidden, const T* __restrict__ delta, long long n) {
    grid_chain_entry();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        hidden[i] += Num<T>::to_f(delta[i]);
}

// hidden += delta over n elements (the residual stream catching up with a pending update).
QF_EXPORT int qf_residual_add(int is_bf16, float* hidden, const void* delta, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const long long most = (long long)(qf_sm_count() > 0 ? qf_sm_count() : 1) * 8;
    const int blocks = (int)((n + 255) / 256 < most ? (n + 255) / 256 : most);
    if (is_bf16)
        return (int)launch_pdl(residual_add_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, hidden, (const bf16*)delta, n);
    return (int)launch_pdl(residual_add_kernel<float>, dim3(blocks), dim3(256), 0, stream, hidden, (const float*)delta, n);
}

// A sublayer's output normalised on its way into the stream, and the stream normalised again for the next sublayer:
//   hidden += y * rsqrt(mean(y^2) + eps_post) * post_weight;   out = hidden * rsqrt(mean(hidden^2) + eps_next) * next_weight
// (the second half only when next_weight is given). Both sums of squares, both roots and the addition are float32. A block
// per row; a thread keeps KEEP of the row's elements in registers between the passes (KEEP x 256 >= width for rows of up to
// 4,096 columns; wider rows are read again).
// With `dest`, row t of y is not stored anywhere: it is the sum of `top` rows y[dest[t * top + k]] (each times
// row_weight[that row], if given), summed in float32 in the order of k: what a mixture of experts leaves per token.
// NSRC is how many rows are summed, known when the kernel is chosen (1, 2, up to 4; 0: any number, by a loop), so that
// a thread's loads of the stream, of y and of both norm weights are few and all on their way together: a step of a few
// rows waits for this kernel's chain of loads, a step of thousands for its bytes, and neither should wait for instructions.
template <typename T, int KEEP, int NSRC>
__global__ void __launch_bounds__(256)
sandwich_norm_kernel(float* __restrict__ hidden, const T* __restrict__ y, const T* __restrict__ post_weight, float eps_post,
                     const T* __restrict__ next_weight, float eps_next, T* __restrict__ out, int width,
                     const int* __restrict__ dest, int top, const float* __restrict__ row_weight) {
    grid_chain_entry();
    __shared__ float scratch[33];
    float* h = hidden + (size_t)blockIdx.x * width;
    constexpr int NS = NSRC > 0 ? NSRC : 1;
    const int n_src = dest ? top : 1;
    const T* src[NS];
    float w[NS];
#pragma unroll
    for (int k = 0; k < NS; ++k) {
        const bool on = NSRC > 0 && k < n_src;
        const int r = on ? (dest ? dest[(size_t)blockIdx.x * top + k] : (int)blockIdx.x) : 0;
        src[k] = y + (size_t)r * width;
        w[k] = on ? ((dest && row_weight) ? row_weight[r] : 1.f) : 0.f;
    }
    auto y_at = [&](int c) -> float {
        float sum = 0.f;
        if (NSRC > 0) {
#pragma unroll
            for (int k = 0; k < NS; ++k) sum += (NSRC <= 2 || k < n_src) ? Num<T>::to_f(src[k][c]) * w[k] : 0.f;
        } else {
            for (int k = 0; k < top; ++k) {
                const int r = dest[(size_t)blockIdx.x * top + k];
                sum += Num<T>::to_f(y[(size_t)r * width + c]) * (row_weight ? row_weight[r] : 1.f);
            }
        }
        return sum;
    };
    float kept[KEEP], hv[KEEP], pw[KEEP], nw[KEEP];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < KEEP; ++u) {
        const int c = threadIdx.x + u * 256;
        const bool ok = c < width;
        hv[u] = ok ? h[c] : 0.f;
        kept[u] = ok ? y_at(c) : 0.f;
        pw[u] = ok ? Num<T>::to_f(post_weight[c]) : 0.f;
        nw[u] = (ok && next_weight) ? Num<T>::to_f(next_weight[c]) : 0.f;
        ss += kept[u] * kept[u];
    }
    for (int c = threadIdx.x + KEEP * 256; c < width; c += 256) {
        const float v = y_at(c);
        ss += v * v;
    }
    const float inv_y = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps_post);
    ss = 0.f;
#pragma unroll
    for (int u = 0; u < KEEP; ++u) {
        const int c = threadIdx.x + u * 256;
        if (c < width) {
            kept[u] = hv[u] + kept[u] * inv_y * pw[u];
            h[c] = kept[u];
            ss += kept[u] * kept[u];
        }
    }
    for (int c = threadIdx.x + KEEP * 256; c < width; c += 256) {
        const float v = h[c] + y_at(c) * inv_y * Num<T>::to_f(post_weight[c]);
        h[c] = v;
        ss += v * v;
    }
    if (!next_weight) return;
    const float inv_h = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps_next);
    T* o = out + (size_t)blockIdx.x * width;
#pragma unroll
    for (int u = 0; u < KEEP; ++u) {
        const int c = threadIdx.x + u * 256;
        if (c < width) o[c] = Num<T>::from_f(kept[u] * inv_h * nw[u]);
    }
    for (int c = threadIdx.x + KEEP * 256; c < width; c += 256)   // each thread re-reads the columns it wrote itself
        o[c] = Num<T>::from_f(h[c] * inv_h * Num<T>::to_f(next_weight[c]));
}

template <typename T, int KEEP>
static int sandwich_launch_keep(float* hidden, const void* y, const void* post_weight, float eps_post, const void* next_weight,
                                float eps_next, void* out, int rows, int width, const int* dest, int top, const float* row_weight,
                                cudaStream_t stream) {
    const int n_src = dest ? top : 1;
#define QF_SANDWICH(NSRC)                                                                                                    \
    return (int)launch_pdl(sandwich_norm_kernel<T, KEEP, NSRC>, dim3(rows), dim3(256), 0, stream, hidden, (const T*)y,       \
                           (const T*)post_weight, eps_post, (const T*)next_weight, eps_next, (T*)out, width, dest, top, row_weight)
    if (n_src == 1) QF_SANDWICH(1);
    if (n_src == 2) QF_SANDWICH(2);
    if (n_src <= 4) QF_SANDWICH(4);
    QF_SANDWICH(0);
#undef QF_SANDWICH
}

// Which kernel runs depends on the width and on the number of rows summed alone, so a row's result does not depend on how
// many rows the step has.
template <typename T>
static int sandwich_launch(float* hidden, const void* y, const void* post_weight, float eps_post, const void* next_weight,
                           float eps_next, void* out, int rows, int width, const int* dest, int top, const float* row_weight,
                           cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (width <= 1024)
        return sandwich_launch_keep<T, 4>(hidden, y, post_weight, eps_post, next_weight, eps_next, out, rows, width, dest, top, row_weight, stream);
    if (width <= 2048)
        return sandwich_launch_keep<T, 8>(hidden, y, post_weight, eps_post, next_weight, eps_next, out, rows, width, dest, top, row_weight, stream);
    return sandwich_launch_keep<T, 16>(hidden, y, post_weight, eps_post, next_weight, eps_next, out, rows, width, dest, top, row_weight, stream);
}

// y, post_weight, next_weight (may be null) and out (null with it) share a dtype; hidden is float32 [rows, width]. dest
// (int32 [rows * top], or null), top and row_weight (float32 per row of y, or null): see above; y then has as many rows
// as dest names.
QF_EXPORT int qf_sandwich_norm(int is_bf16, float* hidden, const void* y, const void* post_weight, float eps_post,
                               const void* next_weight, float eps_next, void* out, int rows, int width, const int* dest, int top,
                               const float* row_weight, cudaStream_t stream) {
    return is_bf16 ? sandwich_launch<bf16>(hidden, y, post_weight, eps_post, next_weight, eps_next, out, rows, width, dest, top, row_weight, stream)
                   : sandwich_launch<float>(hidden, y, post_weight, eps_post, next_weight, eps_next, out, rows, width, dest, top, row_weight, stream);
}

// ------------------------------------------------------------------------------------------------------------------
// Dynamic Tanh in the place of a norm: no mean and no variance, element by element
//   hidden += (a + b) (each if given);  out = tanh(alpha * hidden) * weight + bias
// The sum into the stream and the tanh are float32; `out` has the activation type. Two pending outputs are taken because
// a layer whose sublayers both read the one norm leaves two.
template <typename T>
__global__ void __launch_bounds__(256)
add_dyt_norm_kernel(float* __restrict__ hidden, const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ weight,
                    const T* __restrict__ bias, float alpha, T* __restrict__ out, size_t total, int width) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float v = hidden[i];
        if (a || b) {
            v += (a ? Num<T>::to_f(a[i]) : 0.f) + (b ? Num<T>::to_f(b[i]) : 0.f);
            hidden[i] = v;
        }
        const int c = (int)(i % width);
        out[i] = Num<T>::from_f(fmaf(tanhf(alpha * v), Num<T>::to_f(weight[c]), Num<T>::to_f(bias[c])));
    }
}

// Four elements per thread: width % 4 == 0 and pointers that 16-byte (float32) / 8-byte (bfloat16) accesses can address.
template <typename T>
__global__ void __launch_bounds__(256)
add_dyt_norm_vec_kernel(float* __restrict__ hidden, const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ weight,
                        const T* __restrict__ bias, float alpha, T* __restrict__ out, size_t total4, int width4) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (size_t)gridDim.x * blockDim.x) {
        float4 v = *reinterpret_cast<const float4*>(hidden + i * 4);
        if (a || b) {
            const float4 x = a ? Vec4<T>::load(a + i * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 y = b ? Vec4<T>::load(b + i * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            v.x += x.x + y.x;
            v.y += x.y + y.y;
            v.z += x.z + y.z;
            v.w += x.w + y.w;
            *reinterpret_cast<float4*>(hidden + i * 4) = v;
        }
        const int c = (int)(i % width4) * 4;
        const float4 w = Vec4<T>::load(weight + c), s = Vec4<T>::load(bias + c);
        Vec4<T>::store(out + i * 4, make_float4(fmaf(tanhf(alpha * v.x), w.x, s.x), fmaf(tanhf(alpha * v.y), w.y, s.y),
                                                fmaf(tanhf(alpha * v.z), w.z, s.z), fmaf(tanhf(alpha * v.w), w.w, s.w)));
    }
}

static inline int elementwise_blocks(size_t items) {
    const size_t most = (size_t)(qf_sm_count() > 0 ? qf_sm_count() : 1) * 16;
    const size_t want = (items + 255) / 256;
    return (int)(want < most ? (want ? want : 1) : most);
}

template <typename T>
static int launch_dyt(float* hidden, const void* a, const void* b, const void* weight, const void* bias, float alpha, void* out,
                      int rows, int width, cudaStream_t stream) {
    const size_t total = (size_t)rows * width;
    const uintptr_t all = (uintptr_t)hidden | (uintptr_t)a | (uintptr_t)b | (uintptr_t)weight | (uintptr_t)bias | (uintptr_t)out;
    if (width % 4 == 0 && all % 16 == 0)
        return (int)launch_pdl(add_dyt_norm_vec_kernel<T>, dim3(elementwise_blocks(total / 4)), dim3(256), 0, stream, hidden,
                               (const T*)a, (const T*)b, (const T*)weight, (const T*)bias, alpha, (T*)out, total / 4, width / 4);
    return (int)launch_pdl(add_dyt_norm_kernel<T>, dim3(elementwise_blocks(total)), dim3(256), 0, stream, hidden, (const T*)a,
                           (const T*)b, (const T*)weight, (const T*)bias, alpha, (T*)out, total, width);
}

// hidden: float32 [rows][width], updated in place when a or b is given; a, b, weight, bias, out: activation dtype.
QF_EXPORT int qf_add_dyt_norm(int is_bf16, float* hidden, const void* a, const void* b, const void* weight, const void* bias,
                              float alpha, void* out, int rows, int width, cudaStream_t stream) {
    if (rows <= 0 || width <= 0) return 0;
    return is_bf16 ? launch_dyt<bf16>(hidden, a, b, weight, bias, alpha, out, rows, width, stream)
                   : launch_dyt<float>(hidden, a, b, weight, bias, alpha, out, rows, width, stream);
}

// The same norm for a step of ONE token per sequence, with a token shift behind it in the same kernel: beside `out` it writes
//   shifted = taps[c][0] * (the row's previous out, kept per slot in `state`, zeros for slot < 0) + taps[c][1] * out
// and leaves out (as rounded to the activation type) in the state: what a two-tap causal convolution over `out` would give
// and keep, product by product (fmaf(taps[c][0], previous, 0), then fmaf(taps[c][1], out, that)).
template <typename T>
__global__ void __launch_bounds__(256)
add_dyt_norm_shift_kernel(float* __restrict__ hidden, const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ weight,
                          const T* __restrict__ bias, float alpha, T* __restrict__ out, const float* __restrict__ taps,
                          const int* __restrict__ slots, float* __restrict__ state, long long slot_stride, T* __restrict__ shifted,
                          size_t total, int width) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float v = hidden[i];
        if (a || b) {
            v += (a ? Num<T>::to_f(a[i]) : 0.f) + (b ? Num<T>::to_f(b[i]) : 0.f);
            hidden[i] = v;
        }
        const int c = (int)(i % width), slot = slots[i / width];
        const T h = Num<T>::from_f(fmaf(tanhf(alpha * v), Num<T>::to_f(weight[c]), Num<T>::to_f(bias[c])));
        out[i] = h;
        const float u = Num<T>::to_f(h);
        float* kept = slot >= 0 ? state + slot * slot_stride : nullptr;
        float z = fmaf(taps[2 * c], kept ? kept[c] : 0.f, 0.f);
        z = fmaf(taps[2 * c + 1], u, z);
        shifted[i] = Num<T>::from_f(z);
        if (kept) kept[c] = u;
    }
}

// rows: one token of every sequence; slots int32 [rows]; taps float32 [width][2] (the older input's first); state float32, one
// row of `slot_stride` floats per slot whose first `width` hold the previous out.
QF_EXPORT int qf_add_dyt_norm_shift(int is_bf16, float* hidden, const void* a, const void* b, const void* weight, const void* bias,
                                    float alpha, void* out, const float* taps, const int* slots, float* state, long long slot_stride,
                                    void* shifted, int rows, int width, cudaStream_t stream) {
    if (rows <= 0 || width <= 0) return 0;
    const size_t total = (size_t)rows * width;
    if (is_bf16)
        return (int)launch_pdl(add_dyt_norm_shift_kernel<bf16>, dim3(elementwise_blocks(total)), dim3(256), 0, stream, hidden,
                               (const bf16*)a, (const bf16*)b, (const bf16*)weight, (const bf16*)bias, alpha, (bf16*)out, taps, slots,
                               state, slot_stride, (bf16*)shifted, total, width);
    return (int)launch_pdl(add_dyt_norm_shift_kernel<float>, dim3(elementwise_blocks(total)), dim3(256), 0, stream, hidden,
                           (const float*)a, (const float*)b, (const float*)weight, (const float*)bias, alpha, (float*)out, taps, slots,
                           state, slot_stride, (float*)shifted, total, width);
}

// hidden += (a + b): two pending outputs of one layer, summed with each other first, then into the float32 stream.
template <typename T>
__global__ void __launch_bounds__(256)
residual_add_pair_kernel(float* __restrict__ hidden, const T* __restrict__ a, const T* __restrict__ b, size_t total) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        hidden[i] += (a ? Num<T>::to_f(a[i]) : 0.f) + (b ? Num<T>::to_f(b[i]) : 0.f);
}

QF_EXPORT int qf_residual_add_pair(int is_bf16, float* hidden, const void* a, const void* b, long long n, cudaStream_t stream) {
    if (n <= 0 || (!a && !b)) return 0;
    if (is_bf16)
        return (int)launch_pdl(residual_add_pair_kernel<bf16>, dim3(elementwise_blocks((size_t)n)), dim3(256), 0, stream, hidden,
                               (const bf16*)a, (const bf16*)b, (size_t)n);
    return (int)launch_pdl(residual_add_pair_kernel<float>, dim3(elementwise_blocks((size_t)n)), dim3(256), 0, stream, hidden,
                           (const float*)a, (const float*)b, (size_t)n);
}

// Rows of two float32 streams side by side in the activation dtype, as a product's input:
//   out[t] = [ hidden[t] + (a[t] + b[t]) | other[t] ]     (a, b: pending outputs, each if given; hidden is not changed)
template <typename T>
__global__ void __launch_bounds__(256)
stream_pair_kernel(const float* __restrict__ hidden, const T* __restrict__ a, const T* __restrict__ b,
                   const float* __restrict__ other, T* __restrict__ out, size_t total, int width) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / width, c = i % width;
        float v = hidden[i];
        if (a || b) v += (a ? Num<T>::to_f(a[i]) : 0.f) + (b ? Num<T>::to_f(b[i]) : 0.f);
        out[t * 2 * width + c] = Num<T>::from_f(v);
        out[t * 2 * width + width + c] = Num<T>::from_f(other[i]);
    }
}

QF_EXPORT int qf_stream_pair(int is_bf16, const float* hidden, const void* a, const void* b, const float* other, void* out,
                             int rows, int width, cudaStream_t stream) {
    const size_t total = (size_t)rows * width;
    if (total == 0) return 0;
    if (is_bf16)
        return (int)launch_pdl(stream_pair_kernel<bf16>, dim3(elementwise_blocks(total)), dim3(256), 0, stream, hidden, (const bf16*)a,
                               (const bf16*)b, other, (bf16*)out, total, width);
    return (int)launch_pdl(stream_pair_kernel<float>, dim3(elementwise_blocks(total)), dim3(256), 0, stream, hidden, (const float*)a,
                           (const float*)b, other, (float*)out, total, width);
}

// ------------------------------------------------------------------------------------------------------------------
// Sublayer outputs that enter the stream under a factor each (a residual multiplier, the weights of two mixers that run
// side by side):   hidden += sa * a + sb * b   (b may be absent), then the RMS norm of the stream as above. The products,
// their sum, the addition and the statistics are float32; one order of operations in every kernel below:
//   t = sa * a;  t = fma(sb, b, t);  hidden = hidden + t.
template <typename T>
__device__ __forceinline__ float scaled_terms(const T* a, float sa, const T* b, float sb, size_t i) {
    float t = __fmul_rn(sa, Num<T>::to_f(a[i]));   // (intrinsics: the compiler must not fuse these with the addition after them)
    if (b) t = __fmaf_rn(sb, Num<T>::to_f(b[i]), t);
    return t;
}

template <typename T>
__global__ void __launch_bounds__(256)
add_scaled_rms_norm_kernel(float* __restrict__ hidden, const T* __restrict__ a, float sa, const T* __restrict__ b, float sb,
                           const T* __restrict__ weight, T* __restrict__ out, int width, float eps) {
    grid_chain_entry();
    __shared__ float scratch[33];
    const size_t row0 = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = __fadd_rn(hidden[row0 + c], scaled_terms(a, sa, b, sb, row0 + c));
        hidden[row0 + c] = v;
        ss += v * v;
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        out[row0 + c] = Num<T>::from_f(hidden[row0 + c] * inv * Num<T>::to_f(weight[c]));
}

// Narrow rows (width <= 1024, a multiple of 4, 16-byte aligned): a warp per row, the row in the lanes' registers.
template <typename T>
__global__ void __launch_bounds__(NW_ROWS * 32)
add_scaled_rms_norm_warp_kernel(float* __restrict__ hidden, const T* __restrict__ a, float sa, const T* __restrict__ b, float sb,
                                const T* __restrict__ weight, T* __restrict__ out, int rows, int width, float eps) {
    grid_chain_entry();
    const int row = blockIdx.x * NW_ROWS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const size_t row0 = (size_t)row * width;
    const int n4 = width / 4;
    float4 v[NW_MAX], av[NW_MAX], bv[NW_MAX];
#pragma unroll
    for (int u = 0; u < NW_MAX; ++u) {
        const int c = lane + 32 * u;
        const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
        v[u] = c < n4 ? Vec4<float>::load(hidden + row0 + 4 * c) : zero;
        av[u] = c < n4 ? Vec4<T>::load(a + row0 + 4 * c) : zero;
        bv[u] = (b && c < n4) ? Vec4<T>::load(b + row0 + 4 * c) : zero;
    }
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < NW_MAX; ++u) {
        const int c = lane + 32 * u;
        if (c < n4) {
            float4 t = make_float4(__fmul_rn(sa, av[u].x), __fmul_rn(sa, av[u].y), __fmul_rn(sa, av[u].z), __fmul_rn(sa, av[u].w));
            if (b) t = make_float4(__fmaf_rn(sb, bv[u].x, t.x), __fmaf_rn(sb, bv[u].y, t.y), __fmaf_rn(sb, bv[u].z, t.z), __fmaf_rn(sb, bv[u].w, t.w));
            v[u].x = __fadd_rn(v[u].x, t.x);
            v[u].y = __fadd_rn(v[u].y, t.y);
            v[u].z = __fadd_rn(v[u].z, t.z);
            v[u].w = __fadd_rn(v[u].w, t.w);
            Vec4<float>::store(hidden + row0 + 4 * c, v[u]);
        }
        ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)width + eps);
#pragma unroll
    for (int u = 0; u < NW_MAX; ++u) {
        const int c = lane + 32 * u;
        if (c < n4) {
            const float4 w = Vec4<T>::load(weight + 4 * c);
            Vec4<T>::store(out + row0 + 4 * c, make_float4(v[u].x * inv * w.x, v[u].y * inv * w.y, v[u].z * inv * w.z, v[u].w * inv * w.w));
        }
    }
}

template <typename T>
static int launch_scaled_norm(float* hidden, const void* a, float sa, const void* b, float sb, const void* weight, void* out,
                              int rows, int width, float eps, cudaStream_t stream) {
    const uintptr_t align = (uintptr_t)hidden | (uintptr_t)a | (uintptr_t)b | (uintptr_t)weight | (uintptr_t)out;
    if (width % 4 == 0 && width <= 4 * 32 * NW_MAX && align % 16 == 0)
        return (int)launch_pdl(add_scaled_rms_norm_warp_kernel<T>, dim3((rows + NW_ROWS - 1) / NW_ROWS), dim3(NW_ROWS * 32), 0, stream,
                               hidden, (const T*)a, sa, (const T*)b, sb, (const T*)weight, (T*)out, rows, width, eps);
    return (int)launch_pdl(add_scaled_rms_norm_kernel<T>, dim3(rows), dim3(256), 0, stream, hidden, (const T*)a, sa, (const T*)b, sb,
                           (const T*)weight, (T*)out, width, eps);
}

// hidden float32 [rows][width]; a (required), b (or null), weight, out in the activation type.
QF_EXPORT int qf_add_scaled_rms_norm(int is_bf16, float* hidden, const void* a, float sa, const void* b, float sb,
                                     const void* weight, void* out, int rows, int width, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (!a) return (int)cudaErrorInvalidValue;
    return is_bf16 ? launch_scaled_norm<bf16>(hidden, a, sa, b, sb, weight, out, rows, width, eps, stream)
                   : launch_scaled_norm<float>(hidden, a, sa, b, sb, weight, out, rows, width, eps, stream);
}

template <typename T>
__global__ void __launch_bounds__(256)
residual_add_scaled_kernel(float* __restrict__ hidden, const T* __restrict__ a, float sa, const T* __restrict__ b, float sb,
                           size_t total) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        hidden[i] = __fadd_rn(hidden[i], scaled_terms(a, sa, b, sb, i));
}

QF_EXPORT int qf_residual_add_scaled(int is_bf16, float* hidden, const void* a, float sa, const void* b, float sb, long long n,
                                     cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!a) return (int)cudaErrorInvalidValue;
    if (is_bf16)
        return (int)launch_pdl(residual_add_scaled_kernel<bf16>, dim3(elementwise_blocks((size_t)n)), dim3(256), 0, stream, hidden,
                               (const bf16*)a, sa, (const bf16*)b, sb, (size_t)n);
    return (int)launch_pdl(residual_add_scaled_kernel<float>, dim3(elementwise_blocks((size_t)n)), dim3(256), 0, stream, hidden,
                           (const float*)a, sa, (const float*)b, sb, (size_t)n);
}

// ------------------------------------------------------------------------------------------------------------------
// RMS norms over runs of columns of wider rows, in place: for each of up to two runs (say the query columns and the key
// columns of one projection's output), x[t][col0 .. col0 + width) <- x / sqrt(sum(x^2) / count + eps) * weight. `count` is
// how many of the run's columns carry numbers (columns of padding hold zeros and add nothing to the sum). Statistics and
// scaling are float32. A block per (row, run).
struct ColsRun {
    int col0, width, count;
    const void* weight;
};

template <typename T>
__global__ void __launch_bounds__(128)
rms_norm_cols_kernel(T* __restrict__ x, int ld, ColsRun r0, ColsRun r1, float eps) {
    grid_chain_entry();
    __shared__ float scratch[33];
    const ColsRun r = blockIdx.y == 0 ? r0 : r1;
    T* row = x + (size_t)blockIdx.x * ld + r.col0;
    const T* w = (const T*)r.weight;
    float ss = 0.f;
    for (int c = threadIdx.x; c < r.width; c += blockDim.x) {
        const float v = Num<T>::to_f(row[c]);
        ss += v * v;
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)r.count + eps);
    for (int c = threadIdx.x; c < r.width; c += blockDim.x) row[c] = Num<T>::from_f(Num<T>::to_f(row[c]) * inv * Num<T>::to_f(w[c]));
}

QF_EXPORT int qf_rms_norm_cols(int is_bf16, void* x, int ld, int rows, int n_runs, int col0_a, int width_a, int count_a,
                               const void* weight_a, int col0_b, int width_b, int count_b, const void* weight_b, float eps,
                               cudaStream_t stream) {
    if (rows <= 0 || n_runs <= 0) return 0;
    if (n_runs > 2 || count_a <= 0 || (n_runs == 2 && count_b <= 0)) return (int)cudaErrorInvalidValue;
    const ColsRun a = {col0_a, width_a, count_a, weight_a}, b = {col0_b, width_b, count_b, weight_b};
    if (is_bf16) return (int)launch_pdl(rms_norm_cols_kernel<bf16>, dim3(rows, n_runs), dim3(128), 0, stream, (bf16*)x, ld, a, b, eps);
    return (int)launch_pdl(rms_norm_cols_kernel<float>, dim3(rows, n_runs), dim3(128), 0, stream, (float*)x, ld, a, b, eps);
}

// Rows drawn towards another layer's rows of the same tokens, head by head, in place:
//   x[t][h * x_head + c] <- (1 - lambda) * x[..] + lambda * other[t][h * other_head + c],   c < size   (float32 inside)
template <typename T>
__global__ void __launch_bounds__(256)
mix_rows_kernel(T* __restrict__ x, int ldx, const T* __restrict__ other, int ldo, int heads, int size, int x_head, int other_head,
                float lambda, size_t total) {
    grid_chain_entry();
    const float keep = 1.0f - lambda;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / ((size_t)heads * size);
        const int rest = (int)(i % ((size_t)heads * size)), h = rest / size, c = rest % size;
        T* p = x + t * ldx + (size_t)h * x_head + c;
        const float mine = Num<T>::to_f(*p), theirs = Num<T>::to_f(other[t * ldo + (size_t)h * other_head + c]);
        *p = Num<T>::from_f(fmaf(lambda, theirs, keep * mine));
    }
}

QF_EXPORT int qf_mix_rows(int is_bf16, void* x, int ldx, const void* other, int ldo, int rows, int heads, int size, int x_head,
                          int other_head, float lambda, cudaStream_t stream) {
    const size_t total = (size_t)rows * heads * size;
    if (total == 0) return 0;
    if (is_bf16)
        return (int)launch_pdl(mix_rows_kernel<bf16>, dim3(elementwise_blocks(total)), dim3(256), 0, stream, (bf16*)x, ldx,
                               (const bf16*)other, ldo, heads, size, x_head, other_head, lambda, total);
    return (int)launch_pdl(mix_rows_kernel<float>, dim3(elementwise_blocks(total)), dim3(256), 0, stream, (float*)x, ldx,
                           (const float*)other, ldo, heads, size, x_head, other_head, lambda, total);
}

// ------------------------------------------------------------------------------------------------------------------
// What stands between a q | k | v product and the rotation in a layer that norms q and k over their whole rows, as one
// kernel, in place: for each of up to three runs of columns (q, k, v) of x[t]
//   v <- x + bias                                      (bias may be null; rounded to the activation type, as a product's
//                                                       epilogue would leave it)
//   the mixing run only:  v[h * x_head + c] <- (1 - lambda) v + lambda other[t][h * other_head + c],  c < size
//   count > 0:  v <- v / sqrt(sum(v^2) / count + eps) * weight      (count 0: no norm)
// A block per (row, run). Statistics, mixing and scaling are float32.
struct PrepRun {
    int col0, width, count;
    const void* bias;
    const void* weight;
};
struct PrepMix {
    int run;   // which run mixes (-1: none)
    const void* other;
    int ldo, size, x_head, other_head;
    float lambda;
};

template <typename T>
__global__ void __launch_bounds__(128)
rows_prepare_kernel(T* __restrict__ x, int ld, PrepRun r0, PrepRun r1, PrepRun r2, PrepMix mix, float eps) {
    grid_chain_entry();
    __shared__ float scratch[33];
    const PrepRun r = blockIdx.y == 0 ? r0 : (blockIdx.y == 1 ? r1 : r2);
    T* row = x + (size_t)blockIdx.x * ld + r.col0;
    const T* bias = (const T*)r.bias;
    const bool mixes = mix.run == (int)blockIdx.y;
    const T* other = mixes ? (const T*)mix.other + (size_t)blockIdx.x * mix.ldo : nullptr;
    const float keep = 1.0f - mix.lambda;
    float ss = 0.f;
    for (int c = threadIdx.x; c < r.width; c += blockDim.x) {
        float v = Num<T>::to_f(row[c]);
        if (bias) v = Num<T>::to_f(Num<T>::from_f(v + Num<T>::to_f(bias[c])));
        if (mixes) {
            const int h = c / mix.x_head, cc = c % mix.x_head;
            if (cc < mix.size) v = Num<T>::to_f(Num<T>::from_f(fmaf(mix.lambda, Num<T>::to_f(other[(size_t)h * mix.other_head + cc]), keep * v)));
        }
        if (bias || mixes) row[c] = Num<T>::from_f(v);
        ss += v * v;
    }
    if (r.count <= 0) return;
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)r.count + eps);
    const T* w = (const T*)r.weight;
    // each thread reads back the columns it wrote itself
    for (int c = threadIdx.x; c < r.width; c += blockDim.x) row[c] = Num<T>::from_f(Num<T>::to_f(row[c]) * inv * Num<T>::to_f(w[c]));
}

// runs: n_runs (1..3) records of (col0, width, count, bias, weight) as parallel arrays; mix_run -1 for none.
QF_EXPORT int qf_rows_prepare(int is_bf16, void* x, int ld, int rows, int n_runs, const int* col0, const int* width, const int* count,
                              const void* const* bias, const void* const* weight, int mix_run, const void* other, int ldo,
                              int mix_size, int x_head, int other_head, float lambda, float eps, cudaStream_t stream) {
    if (rows <= 0 || n_runs <= 0) return 0;
    if (n_runs > 3 || mix_run >= n_runs) return (int)cudaErrorInvalidValue;
    PrepRun r[3] = {};
    for (int i = 0; i < n_runs; ++i) {
        r[i] = PrepRun{col0[i], width[i], count[i], bias[i], weight[i]};
        if (count[i] > 0 && !weight[i]) return (int)cudaErrorInvalidValue;
    }
    const PrepMix mix = {mix_run, other, ldo, mix_size, x_head > 0 ? x_head : 1, other_head, lambda};
    if (is_bf16)
        return (int)launch_pdl(rows_prepare_kernel<bf16>, dim3(rows, n_runs), dim3(128), 0, stream, (bf16*)x, ld, r[0], r[1], r[2], mix, eps);
    return (int)launch_pdl(rows_prepare_kernel<float>, dim3(rows, n_runs), dim3(128), 0, stream, (float*)x, ld, r[0], r[1], r[2], mix, eps);
}
