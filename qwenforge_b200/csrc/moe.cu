// Routing of a mixture-of-experts feed-forward, on the device from start to end (no count ever reaches the host, so a
// step with routed experts replays from a captured graph like any other).
//
//   plan     from the router's float32 logits [tokens][experts]: per token the `top` experts with the largest
//            score, the score being sigmoid(logit) or, with `softmax_scores`, the softmax over the experts; the weights
//            are the chosen scores, divided by their sum when `renormalize` is set. The (token, expert) pairs are
//            sorted by expert: rows offsets[e] .. offsets[e+1]-1 of the sorted order belong to expert e, and every
//            expert's rows are cut into tiles of `tile_rows` rows for the grouped product (csrc/grouped_gemm.cu).
//            For a step of few tokens the plan can make the logits itself from the tokens' rows and the router's
//            weights (float32 sums of the products, a warp per logit), which saves a launch where launches are the cost.
//   gather   x_sorted[r] = x[token of r] (* weight of r, when the weight multiplies the expert's input)
//   combine  out[t] = sum over the token's pairs, in the order of its choice, of y_sorted[row of the pair]
//            (* weight, when the weight multiplies the expert's output), summed in float32
//
// One block makes the plan: the work is a few values per token. The order of an expert's rows among themselves is
// whatever the block's atomics gave; no result depends on it, since a row of a product is computed alone.
#include <float.h>

#include "common.cuh"

#define MOE_PLAN_THREADS 1024
#define MOE_MAX_TOP 16

// One token's choice: the `top` experts with the largest scores (the larger logit is the larger score; ties go to the
// lower index) and their weights.
// `bias` (float32 per expert, or null) is added to the logits before anything else looks at them.
__device__ __forceinline__ void moe_choose(const float* z_raw, const float* bias, int n_experts, int top, int softmax_scores,
                                           int renormalize, int* chosen, float* weight) {
    auto z = [&](int e) { return bias ? z_raw[e] + bias[e] : z_raw[e]; };
    float top_z = -FLT_MAX, denom = 1.f;
    if (softmax_scores) {
        for (int e = 0; e < n_experts; ++e) top_z = fmaxf(top_z, z(e));
        denom = 0.f;
        for (int e = 0; e < n_experts; ++e) denom += expf(z(e) - top_z);
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        int best = -1;
        float best_z = -FLT_MAX;
        for (int e = 0; e < n_experts; ++e) {
            bool taken = false;
            for (int j = 0; j < k; ++j) taken |= chosen[j] == e;
            if (!taken && (best < 0 || z(e) > best_z)) {
                best = e;
                best_z = z(e);
            }
        }
        chosen[k] = best;
        weight[k] = softmax_scores ? expf(best_z - top_z) / denom : 1.0f / (1.0f + expf(-best_z));
        total += weight[k];
    }
    if (renormalize)
        for (int k = 0; k < top; ++k) weight[k] /= total;
}

// The choice among groups of neighbouring experts, with a correction that steers the choice and not the weights:
//   s_e = sigmoid(z_e);  c_e = s_e + correction_e (the choice score);  the experts form `group_count` equal groups of
//   neighbours, a group's score is the sum of its two largest c (of its one, in groups of one);  only experts of the
//   `group_keep` groups with the largest scores can be chosen;  among them the `top` largest c;  weights s_e, divided by
//   their sum with `renormalize`.  Ties go to the lower index.  (group_count 1: no groups.)
struct MoeGroups {
    const float* correction;   // float32 [experts] or null
    int count, keep;
};
#define MOE_MAX_GROUPS 64

__device__ __forceinline__ void moe_choose_grouped(const float* z_raw, const float* bias, int n_experts, int top, int renormalize,
                                                   MoeGroups groups, int* chosen, float* weight) {
    auto score = [&](int e) { return 1.0f / (1.0f + expf(-(bias ? z_raw[e] + bias[e] : z_raw[e]))); };
    auto choice = [&](int e) { return groups.correction ? score(e) + groups.correction[e] : score(e); };
    unsigned long long kept = ~0ull;
    const int size = n_experts / groups.count;
    if (groups.count > 1 && groups.keep < groups.count) {
        float group_score[MOE_MAX_GROUPS];
        for (int g = 0; g < groups.count; ++g) {
            float first = -FLT_MAX, second = -FLT_MAX;
            for (int e = g * size; e < (g + 1) * size; ++e) {
                const float c = choice(e);
                if (c > first) {
                    second = first;
                    first = c;
                } else if (c > second) {
                    second = c;
                }
            }
            group_score[g] = size > 1 ? first + second : first;
        }
        kept = 0ull;
        for (int k = 0; k < groups.keep; ++k) {
            int best = -1;
            for (int g = 0; g < groups.count; ++g)
                if (!((kept >> g) & 1ull) && (best < 0 || group_score[g] > group_score[best])) best = g;
            kept |= 1ull << best;
        }
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        int best = -1;
        float best_c = -FLT_MAX;
        for (int e = 0; e < n_experts; ++e) {
            if (groups.count > 1 && !((kept >> (e / size)) & 1ull)) continue;
            bool taken = false;
            for (int j = 0; j < k; ++j) taken |= chosen[j] == e;
            if (taken) continue;
            const float c = choice(e);
            if (best < 0 || c > best_c) {
                best = e;
                best_c = c;
            }
        }
        chosen[k] = best;
        weight[k] = score(best);
        total += weight[k];
    }
    if (renormalize)
        for (int k = 0; k < top; ++k) weight[k] /= total;
}

// Scratch in pair order (pair = token * top + k): pair_expert, pair_weight. Results: dest [pairs] (the row of every pair),
// and in row order sorted_token [pairs], sorted_weight float32 [pairs]; offsets [experts + 1]; tile_group, tile_row0
// [max_tiles]; n_tiles [1].
__global__ void __launch_bounds__(MOE_PLAN_THREADS)
moe_plan_kernel(const float* logits, int n_tokens, int n_experts, int top, int softmax_scores, int renormalize,
                int* __restrict__ pair_expert, float* __restrict__ pair_weight, int* __restrict__ sorted_token,
                float* __restrict__ sorted_weight, int* __restrict__ dest, int* __restrict__ offsets,
                int* __restrict__ tile_group, int* __restrict__ tile_row0, int* __restrict__ n_tiles, int max_tiles,
                int tile_rows, const void* __restrict__ x, const void* __restrict__ router, int width, int x_is_bf16,
                const float* __restrict__ bias, MoeGroups groups) {
    grid_chain_entry();
    extern __shared__ int shared[];
    int* counts = shared;                   // [experts]: rows per expert, then every expert's first row
    int* first_tile = shared + n_experts;   // [experts + 1]
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
    if (x) {  // the router's product first: z[t][e] = sum_c x[t][c] * router[e][c], a warp per logit, kept in shared memory
        float* logits_out = reinterpret_cast<float*>(shared + 2 * n_experts + 1);
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
        for (int i = warp; i < n_tokens * n_experts; i += n_warps) {
            const int t = i / n_experts, e = i % n_experts;
            float sum = 0.f;
            if (x_is_bf16) {
                const bf16* xr = (const bf16*)x + (size_t)t * width;
                const bf16* rr = (const bf16*)router + (size_t)e * width;
                if (width % 8 == 0 && (((uintptr_t)x | (uintptr_t)router) & 15) == 0) {
                    // eight elements per load, and no load waits for a sum: a lane's loads are all on their way at once
                    const uint4* xv = reinterpret_cast<const uint4*>(xr);
                    const uint4* rv = reinterpret_cast<const uint4*>(rr);
                    // four steps of a lane at a time, all their loads asked for before the first product (zeros beyond the
                    // row's end add nothing): the sums run in the same order as one step after the other
                    for (int c0 = lane; c0 < width / 8; c0 += 4 * 32) {
                        uint4 a[4], b[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int c = c0 + 32 * u;
                            a[u] = b[u] = make_uint4(0u, 0u, 0u, 0u);
                            if (c < width / 8) {
                                a[u] = xv[c];
                                b[u] = rv[c];
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            if (c0 + 32 * u >= width / 8) break;
                            const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a[u]);
                            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b[u]);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float2 af = __bfloat1622float2(a2[j]), bf = __bfloat1622float2(b2[j]);
                                sum = fmaf(af.x, bf.x, sum);
                                sum = fmaf(af.y, bf.y, sum);
                            }
                        }
                    }
                } else {
                    for (int c = lane; c < width; c += 32) sum = fmaf(__bfloat162float(xr[c]), __bfloat162float(rr[c]), sum);
                }
            } else {
                const float* xr = (const float*)x + (size_t)t * width;
                const float* rr = (const float*)router + (size_t)e * width;
                for (int c = lane; c < width; c += 32) sum = fmaf(xr[c], rr[c], sum);
            }
            sum = warp_sum(sum);
            if (lane == 0) logits_out[i] = bias ? sum + bias[e] : sum;   // the bias once, here: the choice reads shared memory only
        }
        logits = logits_out;
        bias = nullptr;
    }
    __syncthreads();
    // pass 1: choose, and take a rank among the expert's rows
    for (int t = threadIdx.x; t < n_tokens; t += blockDim.x) {
        int chosen[MOE_MAX_TOP];
        float weight[MOE_MAX_TOP];
        if (groups.count > 0) moe_choose_grouped(logits + (size_t)t * n_experts, bias, n_experts, top, renormalize, groups, chosen, weight);
        else moe_choose(logits + (size_t)t * n_experts, bias, n_experts, top, softmax_scores, renormalize, chosen, weight);
        for (int k = 0; k < top; ++k) {
            const int pair = t * top + k;
            pair_expert[pair] = chosen[k];
            dest[pair] = atomicAdd(&counts[chosen[k]], 1);        // for now: the pair's rank among its expert's rows
            pair_weight[pair] = weight[k];
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int row = 0, tile = 0;
        for (int e = 0; e < n_experts; ++e) {
            const int n = counts[e];
            offsets[e] = row;
            counts[e] = row;
            first_tile[e] = tile;
            row += n;
            tile += (n + tile_rows - 1) / tile_rows;
        }
        offsets[n_experts] = row;
        first_tile[n_experts] = tile;
        n_tiles[0] = tile < max_tiles ? tile : max_tiles;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        const int row0 = counts[e];
        for (int i = first_tile[e]; i < first_tile[e + 1] && i < max_tiles; ++i) {
            tile_group[i] = e;
            tile_row0[i] = row0 + (i - first_tile[e]) * tile_rows;
        }
    }
    // pass 2: every pair's row (each thread finishes the pairs it made itself)
    for (int t = threadIdx.x; t < n_tokens; t += blockDim.x) {
        for (int k = 0; k < top; ++k) {
            const int pair = t * top + k;
            const int row = counts[pair_expert[pair]] + dest[pair];
            dest[pair] = row;
            sorted_token[row] = t;
            sorted_weight[row] = pair_weight[pair];
        }
    }
}

// The same plan for a long step, where one block would be what the step waits for: (1) blocks of 256 tokens choose and count
// in shared memory, then reserve their rows of every expert with ONE atomic per block and expert on `expert_rows` (zero
// before the launch); (2) one block turns the experts' row counts into offsets and tiles; (3) every pair goes to its row.
__global__ void __launch_bounds__(256)
moe_route_kernel(const float* __restrict__ logits, int n_tokens, int n_experts, int top, int softmax_scores, int renormalize,
                 int* __restrict__ pair_expert, float* __restrict__ pair_weight, int* __restrict__ dest,
                 int* __restrict__ expert_rows, const float* __restrict__ bias, MoeGroups groups) {
    grid_chain_entry();
    extern __shared__ int shared[];
    int* counts = shared;               // [experts] pairs of this block
    int* base = shared + n_experts;     // [experts] where this block's pairs start among the expert's rows
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    int chosen[MOE_MAX_TOP], rank[MOE_MAX_TOP];
    float weight[MOE_MAX_TOP];
    if (t < n_tokens) {
        if (groups.count > 0) moe_choose_grouped(logits + (size_t)t * n_experts, bias, n_experts, top, renormalize, groups, chosen, weight);
        else moe_choose(logits + (size_t)t * n_experts, bias, n_experts, top, softmax_scores, renormalize, chosen, weight);
        for (int k = 0; k < top; ++k) rank[k] = atomicAdd(&counts[chosen[k]], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) base[e] = counts[e] > 0 ? atomicAdd(&expert_rows[e], counts[e]) : 0;
    __syncthreads();
    if (t < n_tokens)
        for (int k = 0; k < top; ++k) {
            const int pair = t * top + k;
            pair_expert[pair] = chosen[k];
            dest[pair] = base[chosen[k]] + rank[k];
            pair_weight[pair] = weight[k];
        }
}

__global__ void __launch_bounds__(256)
moe_offsets_kernel(const int* __restrict__ expert_rows, int n_experts, int* __restrict__ offsets, int* __restrict__ tile_group,
                   int* __restrict__ tile_row0, int* __restrict__ n_tiles, int max_tiles, int tile_rows) {
    grid_chain_entry();
    extern __shared__ int shared[];
    int* first_row = shared;                 // [experts]
    int* first_tile = shared + n_experts;    // [experts + 1]
    if (threadIdx.x == 0) {
        int row = 0, tile = 0;
        for (int e = 0; e < n_experts; ++e) {
            const int n = expert_rows[e];
            offsets[e] = row;
            first_row[e] = row;
            first_tile[e] = tile;
            row += n;
            tile += (n + tile_rows - 1) / tile_rows;
        }
        offsets[n_experts] = row;
        first_tile[n_experts] = tile;
        n_tiles[0] = tile < max_tiles ? tile : max_tiles;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x)
        for (int i = first_tile[e]; i < first_tile[e + 1] && i < max_tiles; ++i) {
            tile_group[i] = e;
            tile_row0[i] = first_row[e] + (i - first_tile[e]) * tile_rows;
        }
}

__global__ void __launch_bounds__(256)
moe_place_kernel(const int* __restrict__ pair_expert, const float* __restrict__ pair_weight, const int* __restrict__ offsets,
                 int* __restrict__ dest, int* __restrict__ sorted_token, float* __restrict__ sorted_weight, int pairs, int top) {
    grid_chain_entry();
    const int pair = blockIdx.x * blockDim.x + threadIdx.x;
    if (pair >= pairs) return;
    const int row = offsets[pair_expert[pair]] + dest[pair];
    dest[pair] = row;
    sorted_token[row] = pair / top;
    sorted_weight[row] = pair_weight[pair];
}

template <typename T>
__global__ void __launch_bounds__(128)
moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ sorted_token, const float* __restrict__ sorted_weight,
                  T* __restrict__ out, int n_rows, int width, int scale_input) {
    grid_chain_entry();
    const int r = blockIdx.x;
    if (r >= n_rows) return;
    const T* src = x + (size_t)sorted_token[r] * width;
    const float w = scale_input ? sorted_weight[r] : 1.f;
    T* dst = out + (size_t)r * width;
    if (!scale_input && ((size_t)width * sizeof(T)) % 16 == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0) {
        const uint4* s4 = reinterpret_cast<const uint4*>(src);   // a plain copy of the row, 16 bytes at a time
        uint4* d4 = reinterpret_cast<uint4*>(dst);
        for (int c = threadIdx.x; c < (int)((size_t)width * sizeof(T) / 16); c += blockDim.x) d4[c] = s4[c];
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = Num<T>::from_f(Num<T>::to_f(src[c]) * w);
}

template <typename T>
__global__ void __launch_bounds__(128)
moe_combine_kernel(const T* __restrict__ y, const int* __restrict__ dest, const float* __restrict__ sorted_weight,
                   T* __restrict__ out, int n_tokens, int top, int width, int scale_output, const T* __restrict__ extra,
                   const float* __restrict__ extra_gate, const T* __restrict__ gate_input, const T* __restrict__ gate_weight,
                   int gate_k) {
    grid_chain_entry();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    // an output that every token gets beside its chosen ones (`extra`), under a sigmoid gate of one logit per token: given,
    // or formed here as the token's row times the gate's weights (float32 sums in a fixed order)
    constexpr int V = 16 / (int)sizeof(T);
    // the rows of the token's pairs and their weights are asked for first: two loads that hang on each other, on their way
    // while the gate's logit is formed
    const bool wide = width % V == 0 && top <= MOE_MAX_TOP && (((uintptr_t)y | (uintptr_t)out | (uintptr_t)extra) & 15) == 0;
    int row[MOE_MAX_TOP];
    float rw[MOE_MAX_TOP];
    if (wide) {
#pragma unroll
        for (int k = 0; k < MOE_MAX_TOP; ++k)
            if (k < top) {
                row[k] = dest[t * top + k];
                rw[k] = scale_output ? sorted_weight[row[k]] : 1.f;
            }
    }
    float share = extra ? 1.f : 0.f;
    if (extra && extra_gate) share = 1.f / (1.f + expf(-extra_gate[t]));
    if (extra && gate_weight) {
        float sum = 0.f;
        if (gate_k % V == 0 && (((uintptr_t)gate_input | (uintptr_t)gate_weight) & 15) == 0) {
            for (int c = threadIdx.x * V; c < gate_k; c += blockDim.x * V) {   // 16 bytes of the row and of the weights at a time
                T a[V], b[V];
                *reinterpret_cast<uint4*>(a) = *reinterpret_cast<const uint4*>(gate_input + (size_t)t * gate_k + c);
                *reinterpret_cast<uint4*>(b) = *reinterpret_cast<const uint4*>(gate_weight + c);
#pragma unroll
                for (int v = 0; v < V; ++v) sum = fmaf(Num<T>::to_f(a[v]), Num<T>::to_f(b[v]), sum);
            }
        } else {
            for (int c = threadIdx.x; c < gate_k; c += blockDim.x)
                sum = fmaf(Num<T>::to_f(gate_input[(size_t)t * gate_k + c]), Num<T>::to_f(gate_weight[c]), sum);
        }
        share = 1.f / (1.f + expf(-block_sum(sum, scratch)));
    }
    if (wide) {
        // the same sums, 16 bytes of every row at a time
        for (int c = threadIdx.x * V; c < width; c += blockDim.x * V) {
            float sum[V];
#pragma unroll
            for (int v = 0; v < V; ++v) sum[v] = 0.f;
#pragma unroll
            for (int k = 0; k < MOE_MAX_TOP; ++k)
                if (k < top) {
                    T in[V];
                    *reinterpret_cast<uint4*>(in) = *reinterpret_cast<const uint4*>(y + (size_t)row[k] * width + c);
#pragma unroll
                    for (int v = 0; v < V; ++v) sum[v] += scale_output ? Num<T>::to_f(in[v]) * rw[k] : Num<T>::to_f(in[v]);
                }
            T res[V];
            if (extra) {
                T in[V];
                *reinterpret_cast<uint4*>(in) = *reinterpret_cast<const uint4*>(extra + (size_t)t * width + c);
#pragma unroll
                for (int v = 0; v < V; ++v) sum[v] = fmaf(share, Num<T>::to_f(in[v]), sum[v]);
            }
#pragma unroll
            for (int v = 0; v < V; ++v) res[v] = Num<T>::from_f(sum[v]);
            *reinterpret_cast<uint4*>(out + (size_t)t * width + c) = *reinterpret_cast<const uint4*>(res);
        }
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float sum = 0.f;
        for (int k = 0; k < top; ++k) {
            const int row = dest[t * top + k];
            const float v = Num<T>::to_f(y[(size_t)row * width + c]);
            sum += scale_output ? v * sorted_weight[row] : v;
        }
        if (extra) sum = fmaf(share, Num<T>::to_f(extra[(size_t)t * width + c]), sum);
        out[(size_t)t * width + c] = Num<T>::from_f(sum);
    }
}

// pairs = n_tokens * top: pair_expert, pair_weight (scratch), sorted_token, sorted_weight and dest have that many elements;
// tile_group and tile_row0 max_tiles >= ceil(pairs / tile_rows) + n_experts. Either `logits` float32 [n_tokens][n_experts]
// is given, or x [n_tokens][width] and router [n_experts][width] (both bfloat16 or both float32), from which the kernel makes
// the logits itself in shared memory (n_tokens * n_experts <= 8192).
// bias: float32 [n_experts] added to the logits, or null.
// correction (float32 [n_experts] or null), group_count, group_keep: the choice among groups of neighbouring experts
// (`moe_choose_grouped`; sigmoid scores); group_count 0: the plain choice.
QF_EXPORT int qf_moe_plan_grouped(const float* logits, int n_tokens, int n_experts, int top, int softmax_scores, int renormalize,
                                  int* pair_expert, float* pair_weight, int* sorted_token, float* sorted_weight, int* dest,
                                  int* offsets, int* tile_group, int* tile_row0, int* n_tiles, int max_tiles, int tile_rows,
                                  const void* x, const void* router, int width, int x_is_bf16, const float* bias,
                                  const float* correction, int group_count, int group_keep, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (group_count < 0 || group_count > MOE_MAX_GROUPS || (group_count > 0 && (n_experts % group_count || group_keep < 1 ||
        group_keep > group_count || (long long)group_keep * (n_experts / group_count) < top || softmax_scores)))
        return (int)cudaErrorInvalidValue;
    const MoeGroups groups = {correction, group_count, group_keep};
    if (top < 1 || top > MOE_MAX_TOP || top > n_experts || n_experts > 8192 || tile_rows <= 0) return (int)cudaErrorInvalidValue;
    if (!logits && !(x && router && (long long)n_tokens * n_experts <= 8192)) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)(2 * n_experts + 1) * sizeof(int) + (logits ? 0 : (size_t)n_tokens * n_experts * sizeof(float));
    return (int)launch_pdl(moe_plan_kernel, dim3(1), dim3(MOE_PLAN_THREADS), smem, stream, logits, n_tokens, n_experts, top,
                           softmax_scores, renormalize, pair_expert, pair_weight, sorted_token, sorted_weight, dest, offsets,
                           tile_group, tile_row0, n_tiles, max_tiles, tile_rows, logits ? nullptr : x, router, width, x_is_bf16, bias,
                           groups);
}

QF_EXPORT int qf_moe_plan_biased(const float* logits, int n_tokens, int n_experts, int top, int softmax_scores, int renormalize,
                                 int* pair_expert, float* pair_weight, int* sorted_token, float* sorted_weight, int* dest,
                                 int* offsets, int* tile_group, int* tile_row0, int* n_tiles, int max_tiles, int tile_rows,
                                 const void* x, const void* router, int width, int x_is_bf16, const float* bias,
                                 cudaStream_t stream) {
    return qf_moe_plan_grouped(logits, n_tokens, n_experts, top, softmax_scores, renormalize, pair_expert, pair_weight, sorted_token,
                               sorted_weight, dest, offsets, tile_group, tile_row0, n_tiles, max_tiles, tile_rows, x, router, width,
                               x_is_bf16, bias, nullptr, 0, 0, stream);
}

QF_EXPORT int qf_moe_plan(const float* logits, int n_tokens, int n_experts, int top, int softmax_scores, int renormalize,
                          int* pair_expert, float* pair_weight, int* sorted_token, float* sorted_weight, int* dest,
                          int* offsets, int* tile_group, int* tile_row0, int* n_tiles, int max_tiles, int tile_rows,
                          const void* x, const void* router, int width, int x_is_bf16, cudaStream_t stream) {
    return qf_moe_plan_biased(logits, n_tokens, n_experts, top, softmax_scores, renormalize, pair_expert, pair_weight, sorted_token,
                              sorted_weight, dest, offsets, tile_group, tile_row0, n_tiles, max_tiles, tile_rows, x, router, width,
                              x_is_bf16, nullptr, stream);
}

QF_EXPORT int qf_moe_gather(int is_bf16, const void* x, const int* sorted_token, const float* sorted_weight, void* out,
                            int n_rows, int width, int scale_input, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (is_bf16)
        return (int)launch_pdl(moe_gather_kernel<bf16>, dim3(n_rows), dim3(128), 0, stream, (const bf16*)x, sorted_token,
                               sorted_weight, (bf16*)out, n_rows, width, scale_input);
    return (int)launch_pdl(moe_gather_kernel<float>, dim3(n_rows), dim3(128), 0, stream, (const float*)x, sorted_token,
                           sorted_weight, (float*)out, n_rows, width, scale_input);
}

// extra: [n_tokens][width] added to every token's sum (or null), times sigmoid(extra_gate[t]) where extra_gate (float32
// [n_tokens]) is given, or times sigmoid(gate_input[t] . gate_weight) where gate_weight [gate_k] and gate_input
// [n_tokens][gate_k] are.
QF_EXPORT int qf_moe_combine_shared(int is_bf16, const void* y, const int* dest, const float* sorted_weight, void* out, int n_tokens,
                                    int top, int width, int scale_output, const void* extra, const float* extra_gate,
                                    const void* gate_input, const void* gate_weight, int gate_k, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (is_bf16)
        return (int)launch_pdl(moe_combine_kernel<bf16>, dim3(n_tokens), dim3(128), 0, stream, (const bf16*)y, dest, sorted_weight,
                               (bf16*)out, n_tokens, top, width, scale_output, (const bf16*)extra, extra_gate,
                               (const bf16*)gate_input, (const bf16*)gate_weight, gate_k);
    return (int)launch_pdl(moe_combine_kernel<float>, dim3(n_tokens), dim3(128), 0, stream, (const float*)y, dest, sorted_weight,
                           (float*)out, n_tokens, top, width, scale_output, (const float*)extra, extra_gate,
                           (const float*)gate_input, (const float*)gate_weight, gate_k);
}

QF_EXPORT int qf_moe_combine(int is_bf16, const void* y, const int* dest, const float* sorted_weight, void* out, int n_tokens,
                             int top, int width, int scale_output, cudaStream_t stream) {
    return qf_moe_combine_shared(is_bf16, y, dest, sorted_weight, out, n_tokens, top, width, scale_output, nullptr, nullptr, nullptr,
                                 nullptr, 0, stream);
}

// The plan of a long step by three launches (see moe_route_kernel). expert_rows: int32 [n_experts], zero before the call.
QF_EXPORT int qf_moe_plan_long_grouped(const float* logits, int n_tokens, int n_experts, int top, int softmax_scores,
                                       int renormalize, int* pair_expert, float* pair_weight, int* sorted_token,
                                       float* sorted_weight, int* dest, int* offsets, int* tile_group, int* tile_row0, int* n_tiles,
                                       int max_tiles, int tile_rows, int* expert_rows, const float* bias, const float* correction,
                                       int group_count, int group_keep, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (group_count < 0 || group_count > MOE_MAX_GROUPS || (group_count > 0 && (n_experts % group_count || group_keep < 1 ||
        group_keep > group_count || (long long)group_keep * (n_experts / group_count) < top || softmax_scores)))
        return (int)cudaErrorInvalidValue;
    const MoeGroups groups = {correction, group_count, group_keep};
    if (top < 1 || top > MOE_MAX_TOP || top > n_experts || n_experts > 4096 || tile_rows <= 0 || !logits || !expert_rows)
        return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)(2 * n_experts + 1) * sizeof(int);
    int code = (int)launch_pdl(moe_route_kernel, dim3((n_tokens + 255) / 256), dim3(256), smem, stream, logits, n_tokens, n_experts,
                               top, softmax_scores, renormalize, pair_expert, pair_weight, dest, expert_rows, bias, groups);
    if (code) return code;
    code = (int)launch_pdl(moe_offsets_kernel, dim3(1), dim3(256), smem, stream, (const int*)expert_rows, n_experts, offsets,
                           tile_group, tile_row0, n_tiles, max_tiles, tile_rows);
    if (code) return code;
    const int pairs = n_tokens * top;
    return (int)launch_pdl(moe_place_kernel, dim3((pairs + 255) / 256), dim3(256), 0, stream, (const int*)pair_expert,
                           (const float*)pair_weight, (const int*)offsets, dest, sorted_token, sorted_weight, pairs, top);
}

QF_EXPORT int qf_moe_plan_long_biased(const float* logits, int n_tokens, int n_experts, int top, int softmax_scores,
                                      int renormalize, int* pair_expert, float* pair_weight, int* sorted_token,
                                      float* sorted_weight, int* dest, int* offsets, int* tile_group, int* tile_row0, int* n_tiles,
                                      int max_tiles, int tile_rows, int* expert_rows, const float* bias, cudaStream_t stream) {
    return qf_moe_plan_long_grouped(logits, n_tokens, n_experts, top, softmax_scores, renormalize, pair_expert, pair_weight,
                                    sorted_token, sorted_weight, dest, offsets, tile_group, tile_row0, n_tiles, max_tiles, tile_rows,
                                    expert_rows, bias, nullptr, 0, 0, stream);
}

QF_EXPORT int qf_moe_plan_long(const float* logits, int n_tokens, int n_experts, int top, int softmax_scores, int renormalize,
                               int* pair_expert, float* pair_weight, int* sorted_token, float* sorted_weight, int* dest,
                               int* offsets, int* tile_group, int* tile_row0, int* n_tiles, int max_tiles, int tile_rows,
                               int* expert_rows, cudaStream_t stream) {
    return qf_moe_plan_long_biased(logits, n_tokens, n_experts, top, softmax_scores, renormalize, pair_expert, pair_weight,
                                   sorted_token, sorted_weight, dest, offsets, tile_group, tile_row0, n_tiles, max_tiles, tile_rows,
                                   expert_rows, nullptr, stream);
}
