// After the q/k/v projection: add the projection's bias (if given), rotate queries and keys (split-half rotary, angles in float32),
// write the queries out and append keys and values to the sequence's cache pages.
//   x' [j]        = x[j] * cos(a_j) - x[j + R/2] * sin(a_j)
//   x' [j + R/2]  = x[j + R/2] * cos(a_j) + x[j] * sin(a_j),   a_j = float(pos) * inv_freq[j],  j < R/2
// R (`rot_dim`) may be smaller than the head size; the remaining components pass through.
// inv_freq == nullptr means no rotation at all (another position encoding did its work before).
#include "common.cuh"

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <typename T>
__global__ void rope_cache_kernel(const T* __restrict__ qkv, const T* __restrict__ bias, int qkv_stride, const int* __restrict__ tok_seq,
                                  const int* __restrict__ tok_pos, const int* __restrict__ slots,
                                  const float* __restrict__ inv_freq, int rot_dim, int n_heads, T* __restrict__ q_out,
                                  KvSite<T> site, int write_cache, int* err) {
    grid_chain_entry();
    const int t = blockIdx.x;
    const int D = site.head_dim, KVH = site.kv_heads;
    const int pos = tok_pos[t];
    const int slot = slots[tok_seq[t]];
    const T* row = qkv + (size_t)t * qkv_stride;
    const int half = rot_dim / 2;
    const int pass = D - rot_dim;  // unrotated tail of each head
    const int q_width = n_heads * D, kv_width = KVH * D;

    // cache rows of this token, one pointer per kind; nullptr where nothing is to be written
    const bool cache = write_cache && slot >= 0;
    if (cache && threadIdx.x == 0) {
        if (site.table[(long long)slot * site.table_stride + pos / QF_PAGE] < 0) atomicOr(err, QF_ERR_NO_PAGE);
    }

    // the token's sines and cosines once for all heads
    __shared__ float sin_s[128], cos_s[128];  // rot_dim <= head_dim <= 256
    for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf((float)pos * inv_freq[j], &sin_s[j], &cos_s[j]);
    __syncthreads();
    // work items: (head, j) rotation pairs of q and k heads, then pass-through and value elements
    const int rot_items = (n_heads + KVH) * half;
    for (int i = threadIdx.x; i < rot_items; i += blockDim.x) {
        const int head = i / half, j = i % half;
        const float s = sin_s[j], c = cos_s[j];
        const bool is_q = head < n_heads;
        const int src = is_q ? head * D : q_width + (head - n_heads) * D;
        float x1 = Num<T>::to_f(row[src + j]), x2 = Num<T>::to_f(row[src + j + half]);
        if (bias) {
            x1 += Num<T>::to_f(bias[src + j]);
            x2 += Num<T>::to_f(bias[src + j + half]);
        }
        const float o1 = x1 * c - x2 * s, o2 = x2 * c + x1 * s;
        if (is_q) {
            T* dst = q_out + (size_t)t * q_width + head * D;
            dst[j] = Num<T>::from_f(o1);
            dst[j + half] = Num<T>::from_f(o2);
        } else if (cache) {
            T* dst = kv_row(site, slot, pos, head - n_heads, 0);
            if (dst) {
                dst[j] = Num<T>::from_f(o1);
                dst[j + half] = Num<T>::from_f(o2);
            }
        }
    }
    // components beyond the rotated part
    const int pass_items = (n_heads + KVH) * pass;
    for (int i = threadIdx.x; i < pass_items; i += blockDim.x) {
        const int head = i / pass, j = rot_dim + i % pass;
        const bool is_q = head < n_heads;
        const int src = is_q ? head * D : q_width + (head - n_heads) * D;
        const T value = bias ? Num<T>::from_f(Num<T>::to_f(row[src + j]) + Num<T>::to_f(bias[src + j])) : row[src + j];
        if (is_q) {
            q_out[(size_t)t * q_width + head * D + j] = value;
        } else if (cache) {
            T* dst = kv_row(site, slot, pos, head - n_heads, 0);
            if (dst) dst[j] = value;
        }
    }
    if (cache) {
        for (int i = threadIdx.x; i < kv_width; i += blockDim.x) {
            T* dst = kv_row(site, slot, pos, i / D, 1);
            const int src = q_width + kv_width + i;
            if (dst) dst[i % D] = bias ? Num<T>::from_f(Num<T>::to_f(row[src]) + Num<T>::to_f(bias[src])) : row[src];
        }
    }
}

// The same for bfloat16 with rows that 16-byte accesses can address (head size, rotated part and row stride
// multiples of 8 elements when halved): a block takes RC_TOKENS tokens, a thread eight components at a time.
// OPTS: the pairs of the rotation may be neighbours (`interleaved`: 2j with 2j + 1; a thread then takes sixteen consecutive
// components), and q and k heads may be divided by their root mean square BEFORE the rotation, times a weight per component
// (`eps` >= 0; `q_norm`, `k_norm` or null). The norm wants the whole head rotated (rot_dim == head size) and a number of
// threads per head (rot_dim / 16) that is a power of two: the head's threads are then neighbours in one warp and add their
// sums of squares by shuffles, the same sum in every one of them.
struct RopeVecOpts {
    int interleaved;
    float eps;              // < 0: no norm
    const bf16* q_norm;
    const bf16* k_norm;
};

#define RC_TOKENS 4
template <bool OPTS>
__global__ void __launch_bounds__(256)
rope_cache_vec_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ bias, int qkv_stride, const int* __restrict__ tok_seq,
                      const int* __restrict__ tok_pos, const int* __restrict__ slots, const float* __restrict__ inv_freq,
                      int rot_dim, int n_heads, bf16* __restrict__ q_out, KvSite<bf16> site, int write_cache, int n_tokens,
                      int* err, RopeVecOpts opts) {
    grid_chain_entry();
    const int D = site.head_dim, KVH = site.kv_heads;
    const int half = rot_dim / 2, pass = D - rot_dim;
    const int q_width = n_heads * D, kv_width = KVH * D;
    const int t0 = blockIdx.x * RC_TOKENS, n_here = min(RC_TOKENS, n_tokens - t0);
    __shared__ float sin_s[RC_TOKENS][128], cos_s[RC_TOKENS][128];
    __shared__ int pos_s[RC_TOKENS];
    __shared__ long long page_s[RC_TOKENS];  // element offset of the token's page in the cache, -1: nothing to write
    if (threadIdx.x < n_here) {
        const int t = t0 + threadIdx.x, pos = tok_pos[t], slot = slots[tok_seq[t]];
        pos_s[threadIdx.x] = pos;
        long long offset = -1;
        if (write_cache && slot >= 0) {
            const int page = site.table[(long long)slot * site.table_stride + pos / QF_PAGE];
            if (page < 0) atomicOr(err, QF_ERR_NO_PAGE);
            else offset = (long long)page * site.page_elems + (long long)(pos % QF_PAGE) * D;
        }
        page_s[threadIdx.x] = offset;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_here * half; i += blockDim.x) {
        const int k = i / half, j = i % half;
        sincosf((float)pos_s[k] * inv_freq[j], &sin_s[k][j], &cos_s[k][j]);
    }
    __syncthreads();
    auto load8 = [&](const bf16* p, const bf16* b, float (&v)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            v[2 * e] = f.x;
            v[2 * e + 1] = f.y;
        }
        if (b) {
            const uint4 braw = *reinterpret_cast<const uint4*>(b);
            const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&braw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(bh[e]);
                v[2 * e] += f.x;
                v[2 * e + 1] += f.y;
            }
        }
    };
    auto store8 = [&](bf16* p, const float (&v)[8]) {
        *reinterpret_cast<uint4*>(p) = make_uint4(pack2(v[0], v[1]), pack2(v[2], v[3]), pack2(v[4], v[5]), pack2(v[6], v[7]));
    };
    // work items per token: groups of eight rotation pairs of q and k heads, then groups of eight components that pass
    // through (the unrotated tail of q and k heads, and the values)
    const int rot_groups = (n_heads + KVH) * (half / 8);
    const int pass_groups = (n_heads + KVH) * (pass / 8) + kv_width / 8;
    const int per_token = rot_groups + pass_groups;
    for (int i = threadIdx.x; i < n_here * per_token; i += blockDim.x) {
        const int k = i / per_token, item = i % per_token, t = t0 + k;
        const bf16* row = qkv + (size_t)t * qkv_stride;
        const long long cache_off = page_s[k];
        if (item < rot_groups) {
            const int per_head = half / 8, head = item / per_head, j = (item % per_head) * 8;
            const bool is_q = head < n_heads;
            const int src = is_q ? head * D : q_width + (head - n_heads) * D;
            const bool neighbours = OPTS && opts.interleaved;
            const int ja = neighbours ? 2 * j : j, jb = neighbours ? 2 * j + 8 : j + half;   // the thread's two runs of eight
            float x1[8], x2[8], o1[8], o2[8];
            load8(row + src + ja, bias ? bias + src + ja : nullptr, x1);
            load8(row + src + jb, bias ? bias + src + jb : nullptr, x2);
            if (OPTS && opts.eps >= 0.f) {
                float ss = 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e) ss = fmaf(x1[e], x1[e], ss);
#pragma unroll
                for (int e = 0; e < 8; ++e) ss = fmaf(x2[e], x2[e], ss);
                const int lane = threadIdx.x & 31;
                const unsigned group = per_head >= 32 ? 0xffffffffu : ((1u << per_head) - 1u) << (lane & ~(per_head - 1));
                for (int off = 1; off < per_head; off <<= 1) ss += __shfl_xor_sync(group, ss, off);
                const float before = 1.f / sqrtf(ss / (float)D + opts.eps);
                const bf16* gain = is_q ? opts.q_norm : opts.k_norm;
                float g1[8], g2[8];
                if (gain) {
                    load8(gain + ja, nullptr, g1);
                    load8(gain + jb, nullptr, g2);
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    x1[e] = gain ? x1[e] * before * g1[e] : x1[e] * before;
                    x2[e] = gain ? x2[e] * before * g2[e] : x2[e] * before;
                }
            }
            if (neighbours) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float s1 = sin_s[k][j + e], c1 = cos_s[k][j + e], s2 = sin_s[k][j + 4 + e], c2 = cos_s[k][j + 4 + e];
                    o1[2 * e] = x1[2 * e] * c1 - x1[2 * e + 1] * s1;
                    o1[2 * e + 1] = x1[2 * e + 1] * c1 + x1[2 * e] * s1;
                    o2[2 * e] = x2[2 * e] * c2 - x2[2 * e + 1] * s2;
                    o2[2 * e + 1] = x2[2 * e + 1] * c2 + x2[2 * e] * s2;
                }
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float s = sin_s[k][j + e], c = cos_s[k][j + e];
                    o1[e] = x1[e] * c - x2[e] * s;
                    o2[e] = x2[e] * c + x1[e] * s;
                }
            }
            bf16* dst = nullptr;
            if (is_q) dst = q_out + (size_t)t * q_width + head * D;
            else if (cache_off >= 0) dst = site.base + cache_off + (long long)(head - n_heads) * QF_PAGE * D;
            if (dst) {
                store8(dst + ja, o1);
                store8(dst + jb, o2);
            }
        } else {
            int rest = item - rot_groups;
            const int head_groups = (n_heads + KVH) * (pass / 8);
            float v[8];
            if (rest < head_groups) {
                const int head = rest / (pass / 8), j = rot_dim + (rest % (pass / 8)) * 8;
                const bool is_q = head < n_heads;
                const int src = is_q ? head * D : q_width + (head - n_heads) * D;
                load8(row + src + j, bias ? bias + src + j : nullptr, v);
                if (is_q) store8(q_out + (size_t)t * q_width + head * D + j, v);
                else if (cache_off >= 0) store8(site.base + cache_off + (long long)(head - n_heads) * QF_PAGE * D + j, v);
            } else if (cache_off >= 0) {
                rest -= head_groups;
                const int c = rest * 8, src = q_width + kv_width + c;  // value component c of the token: head c / D
                load8(row + src, bias ? bias + src : nullptr, v);
                store8(site.base + cache_off + (long long)(KVH + c / D) * QF_PAGE * D + c % D, v);
            }
        }
    }
}

template <typename T>
static int launch(const void* qkv, const void* bias, int qkv_stride, const int* tok_seq, const int* tok_pos, const int* slots,
                  const float* inv_freq, int rot_dim, int n_heads, void* q_out, void* base, const int* table,
                  long long page_elems, int table_stride, int kv_heads, int head_dim, int write_cache, int n_tokens,
                  int* err, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    KvSite<T> site{(T*)base, table, page_elems, table_stride, kv_heads, head_dim};
    if (!inv_freq) rot_dim = 0;
    if (sizeof(T) == 2 && head_dim % 16 == 0 && rot_dim % 16 == 0 && qkv_stride % 8 == 0 && head_dim <= 256 &&
        ((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)base | (uintptr_t)bias) % 16 == 0 && page_elems % 8 == 0) {
        return (int)launch_pdl(rope_cache_vec_kernel<false>, dim3((n_tokens + RC_TOKENS - 1) / RC_TOKENS), dim3(256), 0, stream,
            (const bf16*)qkv, (const bf16*)bias, qkv_stride, tok_seq, tok_pos, slots, inv_freq, rot_dim, n_heads, (bf16*)q_out,
            KvSite<bf16>{(bf16*)base, table, page_elems, table_stride, kv_heads, head_dim}, write_cache, n_tokens, err,
            RopeVecOpts{0, -1.f, nullptr, nullptr});
    }
    return (int)launch_pdl(rope_cache_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (const T*)qkv, (const T*)bias, qkv_stride, tok_seq, tok_pos, slots, inv_freq,
                                                       rot_dim, n_heads, (T*)q_out, site, write_cache, err);
}

// qkv: [n_tokens][qkv_stride] with q heads, then k heads, then v heads; bias: [(n_heads + 2 kv_heads) * head_dim] or null; q_out: [n_tokens][n_heads * head_dim].
QF_EXPORT int qf_rope_cache_write(int is_bf16, const void* qkv, const void* bias, int qkv_stride, const int* tok_seq, const int* tok_pos,
                                  const int* slots, const float* inv_freq, int rot_dim, int n_heads, void* q_out,
                                  void* base, const int* table, long long page_elems, int table_stride, int kv_heads,
                                  int head_dim, int write_cache, int n_tokens, int* err, cudaStream_t stream) {
    if (rot_dim < 0 || rot_dim > head_dim || (rot_dim & 1) || rot_dim > 256) return (int)cudaErrorInvalidValue;
    return is_bf16 ? launch<bf16>(qkv, bias, qkv_stride, tok_seq, tok_pos, slots, inv_freq, rot_dim, n_heads, q_out, base,
                                  table, page_elems, table_stride, kv_heads, head_dim, write_cache, n_tokens, err,
                                  stream)
                   : launch<float>(qkv, bias, qkv_stride, tok_seq, tok_pos, slots, inv_freq, rot_dim, n_heads, q_out, base,
                                   table, page_elems, table_stride, kv_heads, head_dim, write_cache, n_tokens, err,
                                   stream);
}

// The same with what other kinds of attention need. Every q and k head may be divided by its root mean square over its
// first `norm_dim` components (eps inside the root; eps < 0: no norm): after the rotation and without a weight, or, with
// `norm_first`, before the rotation and times a weight per component (`q_norm`, `k_norm`: [norm_dim] each, shared by the
// heads). The rotation pairs component j with j + rot_dim / 2, or, with `interleaved`, component 2j with 2j + 1. The rows
// may hold queries only (`has_kv` 0: a layer that reads another layer's keys and values). One warp per (token, head): the
// head's components stay in registers between the rotation and the norm. Value heads are copied (with their bias) as
// they are.
#define RN_MAX_PER_LANE 16   // head sizes up to 512

template <typename T>
__global__ void __launch_bounds__(256)
rope_norm_cache_kernel(const T* __restrict__ qkv, const T* __restrict__ bias, int qkv_stride, const int* __restrict__ tok_seq,
                       const int* __restrict__ tok_pos, const int* __restrict__ slots, const float* __restrict__ inv_freq,
                       int rot_dim, int n_heads, T* __restrict__ q_out, KvSite<T> site, int write_cache, int has_kv,
                       int norm_dim, float eps, int n_tokens, int* err, int interleaved, int norm_first,
                       const T* __restrict__ q_norm, const T* __restrict__ k_norm) {
    grid_chain_entry();
    const int D = site.head_dim, KVH = has_kv ? site.kv_heads : 0;
    const int heads_per_token = n_heads + 2 * KVH;
    const int lane = threadIdx.x & 31;
    const int half = rot_dim / 2;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)n_tokens * heads_per_token) return;
    const int t = (int)(item / heads_per_token), head = (int)(item % heads_per_token);
    const int pos = tok_pos[t], slot = slots[tok_seq[t]];
    const bool is_q = head < n_heads, is_v = head >= n_heads + KVH;
    const int src = head * D;      // q heads, then k heads, then v heads, each D wide
    T* dst = nullptr;
    if (is_q) {
        dst = q_out + (size_t)t * n_heads * D + (size_t)head * D;
    } else if (write_cache && slot >= 0) {
        dst = kv_row(site, slot, pos, is_v ? head - n_heads - KVH : head - n_heads, is_v ? 1 : 0);
        if (!dst && lane == 0) atomicOr(err, QF_ERR_NO_PAGE);
    }
    if (!dst) return;
    const T* row = qkv + (size_t)t * qkv_stride + src;
    const bool normed = !is_v && eps >= 0.f;
    const T* gain = is_q ? q_norm : k_norm;   // the norm's weight, where it has one
    auto raw = [&](int d) { return Num<T>::to_f(row[d]) + (bias ? Num<T>::to_f(bias[src + d]) : 0.f); };
    float before = 1.f;   // what the norm multiplies with when it comes first
    if (normed && norm_first) {
        float sum = 0.f;
        for (int d = lane; d < norm_dim; d += 32) {
            const float v = raw(d);
            sum = fmaf(v, v, sum);
        }
        before = 1.f / sqrtf(warp_sum(sum) / (float)norm_dim + eps);
    }
    // component d as the rotation meets it
    auto entering = [&](int d) {
        float v = raw(d);
        if (normed && norm_first && d < norm_dim) v = v * before * (gain ? Num<T>::to_f(gain[d]) : 1.f);
        return v;
    };
    float x[RN_MAX_PER_LANE];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < RN_MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        x[i] = 0.f;
        if (d >= D) continue;
        float own = entering(d);
        if (!is_v && d < rot_dim) {   // component d turns with its partner
            const bool first = interleaved ? (d & 1) == 0 : d < half;
            const int j = interleaved ? d >> 1 : (d < half ? d : d - half);
            const int partner = interleaved ? d ^ 1 : (d < half ? d + half : d - half);
            const float other = entering(partner);
            float sn, cs;
            sincosf((float)pos * inv_freq[j], &sn, &cs);
            own = first ? own * cs - other * sn : own * cs + other * sn;
        }
        x[i] = own;
        if (d < norm_dim) sum = fmaf(own, own, sum);
    }
    float mult = 1.f;
    if (normed && !norm_first) mult = rsqrtf(warp_sum(sum) / (float)norm_dim + eps);
#pragma unroll
    for (int i = 0; i < RN_MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < D) dst[d] = Num<T>::from_f(x[i] * mult);
    }
}

// q_norm, k_norm: the weights of a norm that comes first ([norm_dim], activation dtype), or null.
QF_EXPORT int qf_rope_norm_cache_write_ex(int is_bf16, const void* qkv, const void* bias, int qkv_stride, const int* tok_seq,
                                          const int* tok_pos, const int* slots, const float* inv_freq, int rot_dim, int n_heads,
                                          void* q_out, void* base, const int* table, long long page_elems, int table_stride,
                                          int kv_heads, int head_dim, int write_cache, int has_kv, int norm_dim, float eps,
                                          int n_tokens, int* err, int interleaved, int norm_first, const void* q_norm,
                                          const void* k_norm, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!inv_freq) rot_dim = 0;
    if (rot_dim < 0 || rot_dim > head_dim || (rot_dim & 1) || head_dim > 32 * RN_MAX_PER_LANE || norm_dim <= 0 || norm_dim > head_dim)
        return (int)cudaErrorInvalidValue;
    // long steps of bfloat16 rows that 16-byte accesses can address: eight components per thread, the angles once per token
    const int per_head = rot_dim / 16;
    const bool norm_fits = eps < 0.f || (norm_first && norm_dim == head_dim && rot_dim == head_dim && per_head >= 1 && per_head <= 32 &&
                                         (per_head & (per_head - 1)) == 0);
    if (is_bf16 && has_kv && n_tokens >= 4 * RC_TOKENS && norm_fits && head_dim % 16 == 0 && rot_dim % 16 == 0 && qkv_stride % 8 == 0 &&
        head_dim <= 256 && page_elems % 8 == 0 &&
        ((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)base | (uintptr_t)bias | (uintptr_t)q_norm | (uintptr_t)k_norm) % 16 == 0) {
        return (int)launch_pdl(rope_cache_vec_kernel<true>, dim3((n_tokens + RC_TOKENS - 1) / RC_TOKENS), dim3(256), 0, stream,
            (const bf16*)qkv, (const bf16*)bias, qkv_stride, tok_seq, tok_pos, slots, inv_freq, rot_dim, n_heads, (bf16*)q_out,
            KvSite<bf16>{(bf16*)base, table, page_elems, table_stride, kv_heads, head_dim}, write_cache, n_tokens, err,
            RopeVecOpts{interleaved, eps, (const bf16*)q_norm, (const bf16*)k_norm});
    }
    const long long items = (long long)n_tokens * (n_heads + (has_kv ? 2 * kv_heads : 0));
    const dim3 grid((unsigned)((items + 7) / 8)), block(256);
    if (is_bf16)
        return (int)launch_pdl(rope_norm_cache_kernel<bf16>, grid, block, 0, stream, (const bf16*)qkv, (const bf16*)bias, qkv_stride,
                               tok_seq, tok_pos, slots, inv_freq, rot_dim, n_heads, (bf16*)q_out,
                               KvSite<bf16>{(bf16*)base, table, page_elems, table_stride, kv_heads, head_dim}, write_cache, has_kv,
                               norm_dim, eps, n_tokens, err, interleaved, norm_first, (const bf16*)q_norm, (const bf16*)k_norm);
    return (int)launch_pdl(rope_norm_cache_kernel<float>, grid, block, 0, stream, (const float*)qkv, (const float*)bias, qkv_stride,
                           tok_seq, tok_pos, slots, inv_freq, rot_dim, n_heads, (float*)q_out,
                           KvSite<float>{(float*)base, table, page_elems, table_stride, kv_heads, head_dim}, write_cache, has_kv,
                           norm_dim, eps, n_tokens, err, interleaved, norm_first, (const float*)q_norm, (const float*)k_norm);
}

QF_EXPORT int qf_rope_norm_cache_write(int is_bf16, const void* qkv, const void* bias, int qkv_stride, const int* tok_seq,
                                       const int* tok_pos, const int* slots, const float* inv_freq, int rot_dim, int n_heads,
                                       void* q_out, void* base, const int* table, long long page_elems, int table_stride,
                                       int kv_heads, int head_dim, int write_cache, int has_kv, int norm_dim, float eps,
                                       int n_tokens, int* err, cudaStream_t stream) {
    return qf_rope_norm_cache_write_ex(is_bf16, qkv, bias, qkv_stride, tok_seq, tok_pos, slots, inv_freq, rot_dim, n_heads, q_out,
                                       base, table, page_elems, table_stride, kv_heads, head_dim, write_cache, has_kv, norm_dim,
                                       eps, n_tokens, err, 0, 0, nullptr, nullptr, stream);
}

// Rows of whole blocks beside a cache: once the last position of a block of `pool` positions has been written, the block's
// row in a second cache (`rows`: one row per block, addressed like positions) becomes the mean of the block's keys and the
// mean of its values AS THE CACHE HOLDS THEM (float32 sums, divided by `pool`, rounded to the cache's type). A block of
// threads per (candidate block of the step, sequence, plane of one kv head's keys or values): a step of q tokens that starts
// at position p completes the blocks floor(p / pool) .. floor((p + q) / pool) - 1. The block's positions are dealt to
// POOL_PARTS groups of threads in turn (position j to group j % POOL_PARTS, each summing its own in rising order), and the
// groups' sums are added in the groups' order: one fixed order of additions for a block, whatever the step that completes it.
#define POOL_PARTS 16

template <typename T>
__global__ void __launch_bounds__(POOL_PARTS * 64)
pool_cache_kernel(const int* __restrict__ cu_q, const int* __restrict__ tok_pos, const int* __restrict__ slots, KvSite<T> site,
                  KvSite<T> rows, int pool, int* err) {
    grid_chain_entry();
    extern __shared__ float pool_parts[];   // [POOL_PARTS][head_dim], and one flag per part behind them
    const int seq = blockIdx.y, slot = slots[seq];
    if (slot < 0) return;
    const int begin = cu_q[seq], len = cu_q[seq + 1] - begin;
    if (len <= 0) return;
    const int start = tok_pos[begin];
    const int b = start / pool + blockIdx.x;
    if ((long long)(b + 1) * pool > (long long)start + len) return;   // not complete after this step
    const int D = site.head_dim;
    const int which = blockIdx.z / site.kv_heads, h = blockIdx.z % site.kv_heads;
    const int lanes = blockDim.x / POOL_PARTS, part = threadIdx.x / lanes, lane = threadIdx.x % lanes;
    int* missing = reinterpret_cast<int*>(pool_parts + POOL_PARTS * D);
    if (threadIdx.x == 0) *missing = 0;
    __syncthreads();
    for (int d0 = 0; d0 < D; d0 += lanes) {
        const int d = d0 + lane;
        float sum = 0.f;
        bool held = true;
#pragma unroll 4
        for (int j = part; j < pool; j += POOL_PARTS) {
            const T* src = kv_row(site, slot, b * pool + j, h, which);
            if (src) { if (d < D) sum += Num<T>::to_f(src[d]); }
            else held = false;
        }
        if (!held) *missing = 1;
        if (d < D) pool_parts[part * D + d] = sum;
    }
    __syncthreads();
    T* dst = kv_row(rows, slot, b, h, which);
    if (!dst || *missing) {
        if (threadIdx.x == 0) atomicOr(err, QF_ERR_NO_PAGE);
        return;
    }
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float sum = pool_parts[d];
#pragma unroll
        for (int p = 1; p < POOL_PARTS; ++p) sum += pool_parts[p * D + d];
        dst[d] = Num<T>::from_f(sum / (float)pool);
    }
}

// max_blocks: the most blocks any sequence of the step can complete (max_q_len / pool + 1).
QF_EXPORT int qf_pool_cache_write(int is_bf16, const int* cu_q, const int* tok_pos, const int* slots, int n_seqs, void* base,
                                  const int* table, long long page_elems, int table_stride, void* rows_base, const int* rows_table,
                                  long long rows_page_elems, int rows_table_stride, int kv_heads, int head_dim, int pool,
                                  int max_blocks, int* err, cudaStream_t stream) {
    if (n_seqs <= 0 || max_blocks <= 0) return 0;
    if (pool <= 0) return (int)cudaErrorInvalidValue;
    const dim3 grid(max_blocks, n_seqs, 2 * kv_heads), block(POOL_PARTS * (head_dim <= 32 ? 32 : 64));
    const size_t smem = (size_t)POOL_PARTS * head_dim * sizeof(float) + sizeof(int);
    if (is_bf16)
        return (int)launch_pdl(pool_cache_kernel<bf16>, grid, block, smem, stream, cu_q, tok_pos, slots,
                               KvSite<bf16>{(bf16*)base, table, page_elems, table_stride, kv_heads, head_dim},
                               KvSite<bf16>{(bf16*)rows_base, rows_table, rows_page_elems, rows_table_stride, kv_heads, head_dim},
                               pool, err);
    return (int)launch_pdl(pool_cache_kernel<float>, grid, block, smem, stream, cu_q, tok_pos, slots,
                           KvSite<float>{(float*)base, table, page_elems, table_stride, kv_heads, head_dim},
                           KvSite<float>{(float*)rows_base, rows_table, rows_page_elems, rows_table_stride, kv_heads, head_dim},
                           pool, err);
}

// The rotation angles of a step, once for all its layers: table[t][j] = (cos, sin) of tok_pos[t] * inv_freq[j], float32,
// the same expression as in the kernels above.
__global__ void rope_table_kernel(const int* __restrict__ tok_pos, const float* __restrict__ inv_freq, int n_tokens, int half,
                                  float2* __restrict__ table) {
    grid_chain_entry();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_tokens * half) return;
    float sn, c;
    sincosf((float)tok_pos[i / half] * inv_freq[i % half], &sn, &c);
    table[i] = make_float2(c, sn);
}

QF_EXPORT int qf_rope_table(const int* tok_pos, const float* inv_freq, int n_tokens, int half, void* table, cudaStream_t stream) {
    if (n_tokens <= 0 || half <= 0) return 0;
    const long long total = (long long)n_tokens * half;
    return (int)launch_pdl(rope_table_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, tok_pos, inv_freq, n_tokens, half, (float2*)table);
}
