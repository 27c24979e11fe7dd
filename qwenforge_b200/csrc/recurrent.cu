// Kernels of the recurrent mixers: a state of fixed size per sequence instead of keys and values per position.
//
//   S <- decay_t S + take_t k_t v_t^T,   y_t = S^T q_t        per head; S is dim x vdim, float32, kept per sequence
//
// A state row of a sequence is `state + slot * slot_stride`; every kernel is told at which float of the row its piece
// starts. A sequence whose slot is -1 (a padding entry of the batch) runs from a zero state and stores nothing.
// Everything is float32 inside; q, k, v, the gate of the output and the convolution's input and output carry the
// activation dtype. A token's result depends on its own sequence only, and on the tokens before it in their order, never
// on how they were cut into steps: every kernel walks a sequence token by token in one fixed order of operations.
#include <float.h>

#include "common.cuh"

// ------------------------------------------------------------------------------------------------------------------
// Exponential gates with a running maximum (the mLSTM's): one block per (sequence, head), GATE_TOKENS tokens at a time.
// Every thread works out its token's two log gates (tanh, logsigmoid); then the first warp runs the maximum through the
// tokens in order, 32 at a time, each lane handing its pair to the chain by shuffle; then every thread forms its token's
// three exponentials. The chain's additions are the same, in the same order, for every cut of the sequence.
#define GATE_TOKENS 256

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

__global__ void __launch_bounds__(GATE_TOKENS)
stabilized_gates_kernel(const float* __restrict__ pre, int pre_stride, const float* __restrict__ bias, float cap,
                        const int* __restrict__ cu_q, const int* __restrict__ slots, int n_seqs, float* __restrict__ state,
                        long long slot_stride, long long m_offset, int n_heads, float* __restrict__ decay,
                        float* __restrict__ take, float* __restrict__ floor_out) {
    grid_chain_entry();
    __shared__ float a_s[GATE_TOKENS], f_s[GATE_TOKENS], before_s[GATE_TOKENS], after_s[GATE_TOKENS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int seq = blockIdx.x / n_heads, head = blockIdx.x % n_heads;
    const int begin = cu_q[seq], end = cu_q[seq + 1], slot = slots[seq];
    float* m_ptr = slot >= 0 ? state + slot * slot_stride + m_offset + head : nullptr;
    float m = m_ptr ? *m_ptr : 0.f;          // the first warp's copy is the one that runs
    const float bi = bias[head], bf = bias[n_heads + head];
    for (int t0 = begin; t0 < end; t0 += GATE_TOKENS) {
        const int t = t0 + threadIdx.x, n_here = min(GATE_TOKENS, end - t0);
        float a = 0.f, f = 0.f;
        if (t < end) {
            a = cap * tanhf((pre[(size_t)t * pre_stride + head] + bi) / cap);
            f = log_sigmoid(cap * tanhf((pre[(size_t)t * pre_stride + n_heads + head] + bf) / cap));
        }
        a_s[threadIdx.x] = a;
        f_s[threadIdx.x] = f;
        __syncthreads();
        if (warp == 0) {
            for (int r0 = 0; r0 < n_here; r0 += 32) {
                const float ar = a_s[r0 + lane], fr = f_s[r0 + lane];
                float m_before = 0.f, m_mine = 0.f;
                const int count = min(32, n_here - r0);
                auto link = [&](int j) {
                    const float aj = __shfl_sync(0xffffffffu, ar, j), fj = __shfl_sync(0xffffffffu, fr, j);
                    const float m_new = fmaxf(fj + m, aj);
                    if (lane == j) {
                        m_before = m;
                        m_mine = m_new;
                    }
                    m = m_new;
                };
                if (count == 32) {   // laid out link after link: the shuffles go ahead, an addition and a maximum per token remain
#pragma unroll
                    for (int j = 0; j < 32; ++j) link(j);
                } else {
                    for (int j = 0; j < count; ++j) link(j);
                }
                before_s[r0 + lane] = m_before;
                after_s[r0 + lane] = m_mine;
            }
        }
        __syncthreads();
        if (t < end) {
            const float m_before = before_s[threadIdx.x], m_mine = after_s[threadIdx.x];
            decay[(size_t)t * n_heads + head] = expf(f + m_before - m_mine);
            take[(size_t)t * n_heads + head] = expf(a - m_mine);
            floor_out[(size_t)t * n_heads + head] = expf(-m_mine);
        }
    }
    if (m_ptr && threadIdx.x == 0) *m_ptr = m;
}

QF_EXPORT int qf_stabilized_gates(const float* pre, int pre_stride, const float* bias, float cap, const int* cu_q,
                                  const int* slots, int n_seqs, float* state, long long slot_stride, long long m_offset,
                                  int n_heads, float* decay, float* take, float* floor_out, cudaStream_t stream) {
    if (n_seqs <= 0 || n_heads <= 0) return 0;
    return (int)launch_pdl(stabilized_gates_kernel, dim3(n_seqs * n_heads), dim3(GATE_TOKENS), 0, stream, pre, pre_stride, bias, cap,
                           cu_q, slots, n_seqs, state, slot_stride, m_offset, n_heads, decay, take, floor_out);
}

// ------------------------------------------------------------------------------------------------------------------
// Gates of a state-space recurrence: dt = softplus(dt_pre + dt_bias), decay = exp(-exp(rate_log) * dt), take = dt.
__global__ void decay_gates_kernel(const float* __restrict__ dt_pre, int stride, const float* __restrict__ dt_bias,
                                   const float* __restrict__ rate_log, int n_tokens, int n_heads, float* __restrict__ decay,
                                   float* __restrict__ take) {
    grid_chain_entry();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_tokens * n_heads) return;
    const int t = i / n_heads, h = i % n_heads;
    const float z = dt_pre[(size_t)t * stride + h] + dt_bias[h];
    const float dt = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));   // log(1 + e^z), written so that no e^z overflows
    decay[i] = expf(-expf(rate_log[h]) * dt);
    take[i] = dt;
}

QF_EXPORT int qf_decay_gates(const float* dt_pre, int stride, const float* dt_bias, const float* rate_log, int n_tokens,
                             int n_heads, float* decay, float* take, cudaStream_t stream) {
    const long long total = (long long)n_tokens * n_heads;
    if (total <= 0) return 0;
    return (int)launch_pdl(decay_gates_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, dt_pre, stride,
                           dt_bias, rate_log, n_tokens, n_heads, decay, take);
}

// ------------------------------------------------------------------------------------------------------------------
// The scan. One block per (sequence, head, 16 columns of S). A half warp works on the 16 columns; the rows of S are dealt
// out to the block's half warps, ROWS to each, and stay in registers from the sequence's first token of the step to its
// last, so the chain of dependent operations per token is ROWS long instead of dim, and a head's state is spread over
// vdim / 16 SMs. Tokens are staged SCAN_TOKENS at a time through shared memory (q and k of the head's group, the 16
// values, the two gates); every half warp leaves its rows' part of y for the staged tokens in shared memory, and after
// the tile the parts are added up in the order of the half warps. The next tile's inputs are fetched into registers
// before a tile is worked on, so their way from memory is hidden.
// The vector n of a matrix memory is one more column whose v is 1 (column index vdim), so a head has
// ceil((vdim + 1) / 16) blocks with it. Rows beyond `dim` hold zeros.
// A load that stays where it is written: the next tile's inputs are asked for BEFORE the work on this tile, and a
// compiler that moved the loads down to their first use would put their way from memory back on the critical path.
__device__ __forceinline__ float load_early(const float* p) {
    float x;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(x) : "l"(p));
    return x;
}
__device__ __forceinline__ float load_early(const bf16* p) {
    unsigned short raw;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(raw) : "l"(p));
    return __uint_as_float((unsigned)raw << 16);
}

#define SCAN_TOKENS 32
#define SCAN_COLS 16

// MODE 0: one decay and one take per (token, head), the output read from the state AFTER the token (the form above).
// MODE 1: a decay per (token, head, row of S) (`decay` is [T][heads * dim]), take 1, the output read after the token:
//         S <- diag(w_t) S + k_t v_t^T,  y_t = S^T q_t.
// MODE 2: the same update, but the output is read BEFORE it and the token's own outer product enters under a learned
//         factor per row (`bonus`, float32 [heads][dim]):  y_t = (S + diag(u) k_t v_t^T)^T q_t,  then the update.
template <typename T, int WARPS, int ROWS, int MODE>
__global__ void __launch_bounds__(32 * WARPS)
outer_state_scan_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k, int k_stride, const T* __restrict__ v,
                        int v_stride, const float* __restrict__ decay, const float* __restrict__ take,
                        const int* __restrict__ cu_q, const int* __restrict__ slots, float* __restrict__ state,
                        long long slot_stride, long long s_offset, long long n_offset, int n_heads, int n_groups, int dim,
                        int vdim, float q_scale, float* __restrict__ y, float* __restrict__ nq, const float* __restrict__ bonus,
                        const float* __restrict__ decay_bias, int decay_kind, float inv_tau) {
    grid_chain_entry();
    extern __shared__ __align__(16) float scan_smem[];
    constexpr int THREADS = 32 * WARPS, PARTS = 2 * WARPS, padded = PARTS * ROWS;   // padded >= dim
    float* q_s = scan_smem;                                          // [SCAN_TOKENS][padded]
    float* k_s = q_s + SCAN_TOKENS * padded;                         // [SCAN_TOKENS][padded]
    float* v_s = k_s + SCAN_TOKENS * padded;                         // [SCAN_TOKENS][SCAN_COLS]
    float* part_s = v_s + SCAN_TOKENS * SCAN_COLS;                   // [PARTS][SCAN_TOKENS][SCAN_COLS]
    float* decay_s = part_s + PARTS * SCAN_TOKENS * SCAN_COLS;       // [SCAN_TOKENS]
    float* take_s = decay_s + SCAN_TOKENS;                           // [SCAN_TOKENS]
    float* w_s = take_s + SCAN_TOKENS;                               // [SCAN_TOKENS][padded], MODE 1 and 2: a decay per row
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, head = blockIdx.y, seq = blockIdx.z;
    const int c16 = lane & 15, part = warp * 2 + (lane >> 4);
    const int col = blockIdx.x * SCAN_COLS + c16;           // column of S; vdim is the column of n
    const bool is_n = n_offset >= 0 && col == vdim, active = col < vdim || is_n;
    const int group = head / (n_heads / n_groups);
    const int begin = cu_q[seq], end = cu_q[seq + 1], slot = slots[seq];
    if (begin >= end) return;
    const int d0 = part * ROWS;                             // this half warp's rows of S

    float* column = nullptr;    // the lane's column in the state row: element d at column[d * pitch]
    int pitch = 0;
    if (slot >= 0 && active) {
        float* row = state + slot * slot_stride;
        column = is_n ? row + n_offset + (long long)head * dim : row + s_offset + (long long)head * dim * vdim + col;
        pitch = is_n ? 1 : vdim;
    }
    float s[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) s[r] = (column && d0 + r < dim) ? column[(size_t)(d0 + r) * pitch] : 0.f;

    // A tile's inputs are fetched into registers while the tile before is worked on, and put into shared memory when that
    // one is done: a thread holds ROWS elements of q and of k (SCAN_TOKENS * padded / THREADS), one or two of v, a gate.
    constexpr int QK_EACH = SCAN_TOKENS * padded / THREADS;
    constexpr int V_EACH = (SCAN_TOKENS * SCAN_COLS + THREADS - 1) / THREADS;
    float q_next[QK_EACH], k_next[QK_EACH], v_next[V_EACH], gate_next[2] = {0.f, 0.f};
    float w_next[MODE != 0 ? QK_EACH : 1], u_row[MODE == 2 ? ROWS : 1], bias_row[MODE != 0 ? QK_EACH : 1];
    if constexpr (MODE != 0) {   // the bias of the decays this thread will turn: its elements sit at fixed rows of S
#pragma unroll
        for (int u = 0; u < QK_EACH; ++u) {
            const int d = (threadIdx.x + u * THREADS) % padded;
            bias_row[u] = (decay_kind != 0 && d < dim) ? decay_bias[(size_t)head * dim + d] : 0.f;
        }
    }
    if constexpr (MODE == 2) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) u_row[r] = d0 + r < dim ? bonus[(size_t)head * dim + d0 + r] : 0.f;
    }
    auto fetch = [&](int t0) {
        const int n_here = min(SCAN_TOKENS, end - t0);
#pragma unroll
        for (int u = 0; u < QK_EACH; ++u) {
            const int i = threadIdx.x + u * THREADS, j = i / padded, d = i % padded;
            const bool there = j < n_here && d < dim;
            const size_t t = t0 + j;
            q_next[u] = there ? load_early(q + t * q_stride + group * dim + d) * q_scale : 0.f;
            k_next[u] = there ? load_early(k + t * k_stride + group * dim + d) : 0.f;
            if constexpr (MODE != 0) w_next[u] = there ? load_early(decay + t * ((size_t)n_heads * dim) + (size_t)head * dim + d) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < V_EACH; ++u) {
            const int i = threadIdx.x + u * THREADS, j = i / SCAN_COLS, c = blockIdx.x * SCAN_COLS + i % SCAN_COLS;
            v_next[u] = 0.f;
            if (i < SCAN_TOKENS * SCAN_COLS && j < n_here)
                v_next[u] = c < vdim ? load_early(v + (size_t)(t0 + j) * v_stride + head * vdim + c) : 1.f;
        }
        if (MODE == 0 && threadIdx.x < n_here) {
            gate_next[0] = load_early(decay + (size_t)(t0 + threadIdx.x) * n_heads + head);
            gate_next[1] = load_early(take + (size_t)(t0 + threadIdx.x) * n_heads + head);
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int u = 0; u < QK_EACH; ++u) {
            q_s[threadIdx.x + u * THREADS] = q_next[u];
            k_s[threadIdx.x + u * THREADS] = k_next[u];
            if constexpr (MODE != 0) {
                // the decay itself, or its pre-activation, turned into the decay here, where the load has long arrived (in `fetch`
                // the arithmetic would wait for it): exp(-exp(z + b)) (kind 1), sigmoid(z + b)^(1 / tau) (kind 2); padding stays 0
                float w = w_next[u];
                const int d = (threadIdx.x + u * THREADS) % padded;
                if (decay_kind != 0 && d < dim) {
                    const float z = w + bias_row[u];
                    w = decay_kind == 1 ? expf(-expf(z)) : expf(log_sigmoid(z) * inv_tau);
                }
                w_s[threadIdx.x + u * THREADS] = w;
            }
        }
#pragma unroll
        for (int u = 0; u < V_EACH; ++u) {
            const int i = threadIdx.x + u * THREADS;
            if (i < SCAN_TOKENS * SCAN_COLS) v_s[i] = v_next[u];
        }
        if (threadIdx.x < SCAN_TOKENS) {
            decay_s[threadIdx.x] = gate_next[0];
            take_s[threadIdx.x] = gate_next[1];
        }
    };

    fetch(begin);
    for (int t0 = begin; t0 < end; t0 += SCAN_TOKENS) {
        const int n_here = min(SCAN_TOKENS, end - t0);
        __syncthreads();   // the tile before is summed and written
        stash();
        __syncthreads();
        if (t0 + SCAN_TOKENS < end) fetch(t0 + SCAN_TOKENS);   // on its way while this tile is worked on
        auto token_rows = [&](int j) -> float {   // MODE 1 and 2: one token's update of this half warp's rows, and their part of y
            if constexpr (MODE != 0) {
                const float add = v_s[j * SCAN_COLS + c16];
                const float* kj = k_s + j * padded + d0;
                const float* qj = q_s + j * padded + d0;
                const float* wj = w_s + j * padded + d0;
                float4 kk[ROWS / 4], qq[ROWS / 4], ww[ROWS / 4];
#pragma unroll
                for (int r = 0; r < ROWS / 4; ++r) {
                    kk[r] = *reinterpret_cast<const float4*>(kj + 4 * r);
                    qq[r] = *reinterpret_cast<const float4*>(qj + 4 * r);
                    ww[r] = *reinterpret_cast<const float4*>(wj + 4 * r);
                }
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int r = 0; r < ROWS / 4; ++r) {
                    const float kr[4] = {kk[r].x, kk[r].y, kk[r].z, kk[r].w}, qr[4] = {qq[r].x, qq[r].y, qq[r].z, qq[r].w};
                    const float wr[4] = {ww[r].x, ww[r].y, ww[r].z, ww[r].w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float kv = add * kr[e];
                        if constexpr (MODE == 2) {
                            acc[e] = fmaf(fmaf(u_row[4 * r + e], kv, s[4 * r + e]), qr[e], acc[e]);
                            s[4 * r + e] = fmaf(s[4 * r + e], wr[e], kv);
                        } else {
                            s[4 * r + e] = fmaf(s[4 * r + e], wr[e], kv);
                            acc[e] = fmaf(s[4 * r + e], qr[e], acc[e]);
                        }
                    }
                }
                return (acc[0] + acc[1]) + (acc[2] + acc[3]);
            }
            return 0.f;
        };
        auto token = [&](int j) {
            const float keep = decay_s[j], add = take_s[j] * v_s[j * SCAN_COLS + c16];
            const float* kj = k_s + j * padded + d0;
            const float* qj = q_s + j * padded + d0;
            float4 kk[ROWS / 4], qq[ROWS / 4];   // all of the token's rows asked for at once: one wait, not one per four rows
#pragma unroll
            for (int r = 0; r < ROWS / 4; ++r) {
                kk[r] = *reinterpret_cast<const float4*>(kj + 4 * r);
                qq[r] = *reinterpret_cast<const float4*>(qj + 4 * r);
            }
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int r = 0; r < ROWS / 4; ++r) {
                s[4 * r] = fmaf(add, kk[r].x, s[4 * r] * keep);
                s[4 * r + 1] = fmaf(add, kk[r].y, s[4 * r + 1] * keep);
                s[4 * r + 2] = fmaf(add, kk[r].z, s[4 * r + 2] * keep);
                s[4 * r + 3] = fmaf(add, kk[r].w, s[4 * r + 3] * keep);
                a0 = fmaf(s[4 * r], qq[r].x, a0);
                a1 = fmaf(s[4 * r + 1], qq[r].y, a1);
                a2 = fmaf(s[4 * r + 2], qq[r].z, a2);
                a3 = fmaf(s[4 * r + 3], qq[r].w, a3);
            }
            part_s[(part * SCAN_TOKENS + j) * SCAN_COLS + c16] = (a0 + a1) + (a2 + a3);
        };
        if constexpr (MODE != 0) {
            if (n_here == SCAN_TOKENS) {
                // a whole tile: the tokens' parts of y stay in registers until the tile is done, so that no store stands between
                // one token's loads from shared memory and the next one's and the loads run ahead of the chain of updates
                float parts[SCAN_TOKENS];
#pragma unroll
                for (int j = 0; j < SCAN_TOKENS; ++j) parts[j] = token_rows(j);
#pragma unroll
                for (int j = 0; j < SCAN_TOKENS; ++j) part_s[(part * SCAN_TOKENS + j) * SCAN_COLS + c16] = parts[j];
            } else {
                for (int j = 0; j < n_here; ++j) part_s[(part * SCAN_TOKENS + j) * SCAN_COLS + c16] = token_rows(j);
            }
        } else if (n_here == SCAN_TOKENS) {   // a whole tile: the tokens' code laid out one after another, addresses as constants
#pragma unroll
            for (int j = 0; j < SCAN_TOKENS; ++j) token(j);
        } else {
            for (int j = 0; j < n_here; ++j) token(j);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < n_here * SCAN_COLS; i += THREADS) {   // the parts in the order of the half warps
            const int j = i / SCAN_COLS, c = blockIdx.x * SCAN_COLS + i % SCAN_COLS;
            float sum = 0.f;
#pragma unroll 4
            for (int w = 0; w < PARTS; ++w) sum += part_s[(w * SCAN_TOKENS + j) * SCAN_COLS + i % SCAN_COLS];
            const size_t t = t0 + j;
            if (c < vdim) y[t * ((size_t)n_heads * vdim) + head * vdim + c] = sum;
            else if (n_offset >= 0 && c == vdim) nq[t * n_heads + head] = sum;
        }
    }
    if (column) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
            if (d0 + r < dim) column[(size_t)(d0 + r) * pitch] = s[r];
    }
}

template <typename T, int WARPS, int ROWS, int MODE>
static int launch_scan(const void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride, const float* decay,
                       const float* take, const int* cu_q, const int* slots, int n_seqs, float* state, long long slot_stride,
                       long long s_offset, long long n_offset, int n_heads, int n_groups, int dim, int vdim, float q_scale,
                       float* y, float* nq, const float* bonus, const float* decay_bias, int decay_kind, float inv_tau,
                       cudaStream_t stream) {
    const int columns = vdim + (n_offset >= 0 ? 1 : 0);
    constexpr int PARTS = 2 * WARPS, padded = PARTS * ROWS;
    const size_t smem = (size_t)((MODE != 0 ? 3 : 2) * SCAN_TOKENS * padded + SCAN_TOKENS * SCAN_COLS + PARTS * SCAN_TOKENS * SCAN_COLS + 2 * SCAN_TOKENS) * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(outer_state_scan_kernel<T, WARPS, ROWS, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return (int)launch_pdl(outer_state_scan_kernel<T, WARPS, ROWS, MODE>, dim3((columns + SCAN_COLS - 1) / SCAN_COLS, n_heads, n_seqs),
                           dim3(32 * WARPS), smem, stream, (const T*)q, q_stride, (const T*)k, k_stride, (const T*)v, v_stride, decay,
                           take, cu_q, slots, state, slot_stride, s_offset, n_offset, n_heads, n_groups, dim, vdim, q_scale, y, nq, bonus, decay_bias,
                           decay_kind, inv_tau);
}

#define QF_SCAN_ARGS q, q_stride, k, k_stride, v, v_stride, decay, take, cu_q, slots, n_seqs, state, slot_stride, s_offset, \
                     n_offset, n_heads, n_groups, dim, vdim, q_scale, y, nq, bonus, decay_bias, decay_kind, inv_tau, stream
// 2 * WARPS half warps of ROWS rows each cover `dim` rows
#define QF_SCAN_CASE(WARPS, ROWS) \
    if (dim <= 2 * WARPS * ROWS)  \
        return is_bf16 ? launch_scan<bf16, WARPS, ROWS, MODE>(QF_SCAN_ARGS) : launch_scan<float, WARPS, ROWS, MODE>(QF_SCAN_ARGS);

// q, k: [T][groups * dim] with row strides; v: [T][heads * vdim]; decay, take: float32 [T][heads]; y: float32 [T][heads * vdim];
// nq: float32 [T][heads] or null (then n_offset < 0). State pieces: S [heads][dim][vdim] at s_offset, n [heads][dim] at n_offset.
QF_EXPORT int qf_outer_state_scan(int is_bf16, const void* q, int q_stride, const void* k, int k_stride, const void* v,
                                  int v_stride, const float* decay, const float* take, const int* cu_q, const int* slots,
                                  int n_seqs, float* state, long long slot_stride, long long s_offset, long long n_offset,
                                  int n_heads, int n_groups, int dim, int vdim, float q_scale, float* y, float* nq,
                                  cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (dim <= 0 || vdim <= 0 || n_groups <= 0 || n_heads % n_groups || (n_offset >= 0 && !nq)) return (int)cudaErrorInvalidValue;
    constexpr int MODE = 0;
    const float* bonus = nullptr;
    const float* decay_bias = nullptr;
    const int decay_kind = 0;
    const float inv_tau = 1.f;
    QF_SCAN_CASE(4, 4)
    QF_SCAN_CASE(8, 4)
    QF_SCAN_CASE(16, 4)
    QF_SCAN_CASE(16, 8)
    return (int)cudaErrorInvalidValue;
}

template <int MODE>
static int scan_rows(int is_bf16, const void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride,
                     const float* decay, const int* cu_q, const int* slots, int n_seqs, float* state, long long slot_stride,
                     long long s_offset, int n_heads, int n_groups, int dim, int vdim, float q_scale, float* y, const float* bonus,
                     const float* decay_bias, int decay_kind, float inv_tau, cudaStream_t stream) {
    const float* take = nullptr;
    float* nq = nullptr;
    const long long n_offset = -1;
    QF_SCAN_CASE(4, 4)
    QF_SCAN_CASE(8, 4)
    QF_SCAN_CASE(16, 4)
    QF_SCAN_CASE(16, 8)
    return (int)cudaErrorInvalidValue;
}

// The scan with a decay per row of S: decay is float32 [T][heads * dim]; `bonus` null: the output is read after the token's
// update (MODE 1); `bonus` float32 [heads][dim]: before it, the token's own outer product entering under the bonus (MODE 2).
// decay_kind 0: `decay` holds the decays; 1 and 2: it holds their pre-activations z and the kernel forms exp(-exp(z + b)) or
// sigmoid(z + b)^(1 / tau) on its way in (b = decay_bias, float32 [heads * dim]; the arithmetic of `channel_decay_kernel`).
QF_EXPORT int qf_outer_state_scan_rows(int is_bf16, const void* q, int q_stride, const void* k, int k_stride, const void* v,
                                       int v_stride, const float* decay, const int* cu_q, const int* slots, int n_seqs,
                                       float* state, long long slot_stride, long long s_offset, int n_heads, int n_groups, int dim,
                                       int vdim, float q_scale, float* y, const float* bonus, const float* decay_bias,
                                       int decay_kind, float inv_tau, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (dim <= 0 || vdim <= 0 || n_groups <= 0 || n_heads % n_groups || !decay || decay_kind < 0 || decay_kind > 2 ||
        (decay_kind != 0 && !decay_bias))
        return (int)cudaErrorInvalidValue;
    if (bonus)
        return scan_rows<2>(is_bf16, q, q_stride, k, k_stride, v, v_stride, decay, cu_q, slots, n_seqs, state, slot_stride, s_offset,
                            n_heads, n_groups, dim, vdim, q_scale, y, bonus, decay_bias, decay_kind, inv_tau, stream);
    return scan_rows<1>(is_bf16, q, q_stride, k, k_stride, v, v_stride, decay, cu_q, slots, n_seqs, state, slot_stride, s_offset,
                        n_heads, n_groups, dim, vdim, q_scale, y, bonus, decay_bias, decay_kind, inv_tau, stream);
}

// ------------------------------------------------------------------------------------------------------------------
// A decay per channel from its pre-activation, float32 in and out:
//   kind 0:  w = exp(-exp(z + b))                 (a decay that a low-rank product and a learned offset set)
//   kind 1:  w = sigmoid(z + b)^(1 / tau) = exp(logsigmoid(z + b) * inv_tau)
__global__ void __launch_bounds__(256)
channel_decay_kernel(const float* __restrict__ pre, int stride, const float* __restrict__ bias, int channels, size_t total, int kind,
                     float inv_tau, float* __restrict__ out) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / channels;
        const int c = (int)(i % channels);
        const float z = pre[t * stride + c] + (bias ? bias[c] : 0.f);
        out[i] = kind == 0 ? expf(-expf(z)) : expf(log_sigmoid(z) * inv_tau);
    }
}

QF_EXPORT int qf_channel_decay(const float* pre, int stride, const float* bias, int n_tokens, int channels, int kind, float inv_tau,
                               float* out, cudaStream_t stream) {
    const size_t total = (size_t)n_tokens * channels;
    if (total == 0) return 0;
    if (kind < 0 || kind > 1) return (int)cudaErrorInvalidValue;
    const size_t most = (size_t)(qf_sm_count() > 0 ? qf_sm_count() : 1) * 16, want = (total + 255) / 256;
    return (int)launch_pdl(channel_decay_kernel, dim3((unsigned)(want < most ? want : most)), dim3(256), 0, stream, pre, stride, bias,
                           channels, total, kind, inv_tau, out);
}

// ------------------------------------------------------------------------------------------------------------------
// Token shift into several mixes at once: with h' the row of the token before (the sequence's kept row for its first token
// of the step, zeros at its start), mix s of token t is  h_t + (h'_t - h_t) * mu[s]  (float32 inside), written to
// out[t][s * width ..]. The kept row (float32 [width] at `offset` of the slot's state) then takes the sequence's last h.
// In a step of one token per sequence (`single`) the thread that read a kept element also replaces it; otherwise a second
// kernel does, after every block of the first has read.
template <typename T>
__global__ void __launch_bounds__(256)
shift_mix_kernel(const T* __restrict__ h, int h_stride, const float* __restrict__ mu, int n_mixes, const int* __restrict__ cu_q,
                 const int* __restrict__ tok_seq, const int* __restrict__ slots, float* __restrict__ state, long long slot_stride,
                 long long offset, int width, size_t total, T* __restrict__ out, int single) {
    grid_chain_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / width;
        const int c = (int)(i % width);
        const int seq = tok_seq[t], at = (int)t - cu_q[seq];
        const float mine = Num<T>::to_f(h[t * h_stride + c]);
        float before = 0.f;
        if (at > 0) {
            before = Num<T>::to_f(h[(t - 1) * h_stride + c]);
        } else {
            const int slot = slots[seq];
            if (slot >= 0) {
                float* kept = state + slot * slot_stride + offset + c;
                before = *kept;
                if (single) *kept = mine;
            }
        }
        const float diff = before - mine;
        for (int s = 0; s < n_mixes; ++s)
            out[t * ((size_t)n_mixes * width) + (size_t)s * width + c] = Num<T>::from_f(fmaf(diff, mu[(size_t)s * width + c], mine));
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
shift_keep_kernel(const T* __restrict__ h, int h_stride, const int* __restrict__ cu_q, const int* __restrict__ slots, int n_seqs,
                  float* __restrict__ state, long long slot_stride, long long offset, int width) {
    grid_chain_entry();
    const size_t total = (size_t)n_seqs * width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int seq = (int)(i / width), c = (int)(i % width);
        const int slot = slots[seq], end = cu_q[seq + 1];
        if (slot < 0 || end <= cu_q[seq]) continue;
        state[slot * slot_stride + offset + c] = Num<T>::to_f(h[(size_t)(end - 1) * h_stride + c]);
    }
}

template <typename T>
static int launch_shift_mix(const void* h, int h_stride, const float* mu, int n_mixes, const int* cu_q, const int* tok_seq,
                            const int* slots, int n_seqs, float* state, long long slot_stride, long long offset, int n_tokens,
                            int width, void* out, int single, cudaStream_t stream) {
    const size_t total = (size_t)n_tokens * width, most = (size_t)(qf_sm_count() > 0 ? qf_sm_count() : 1) * 16;
    size_t want = (total + 255) / 256;
    int code = (int)launch_pdl(shift_mix_kernel<T>, dim3((unsigned)(want < most ? want : most)), dim3(256), 0, stream, (const T*)h,
                               h_stride, mu, n_mixes, cu_q, tok_seq, slots, state, slot_stride, offset, width, total, (T*)out, single);
    if (code || single) return code;
    want = ((size_t)n_seqs * width + 255) / 256;
    return (int)launch_pdl(shift_keep_kernel<T>, dim3((unsigned)(want < most ? want : most)), dim3(256), 0, stream, (const T*)h,
                           h_stride, cu_q, slots, n_seqs, state, slot_stride, offset, width);
}

// h: [T][width] with a row stride; mu: float32 [n_mixes][width]; out: [T][n_mixes * width]; state float32 rows per slot.
// single: 1 only if every sequence of the step brings exactly one token.
QF_EXPORT int qf_shift_mix(int is_bf16, const void* h, int h_stride, const float* mu, int n_mixes, const int* cu_q,
                           const int* tok_seq, const int* slots, int n_seqs, float* state, long long slot_stride, long long offset,
                           int n_tokens, int width, void* out, int single, cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (n_mixes <= 0 || width <= 0) return (int)cudaErrorInvalidValue;
    return is_bf16 ? launch_shift_mix<bf16>(h, h_stride, mu, n_mixes, cu_q, tok_seq, slots, n_seqs, state, slot_stride, offset, n_tokens,
                                            width, out, single, stream)
                   : launch_shift_mix<float>(h, h_stride, mu, n_mixes, cu_q, tok_seq, slots, n_seqs, state, slot_stride, offset,
                                             n_tokens, width, out, single, stream);
}

// ------------------------------------------------------------------------------------------------------------------
// What follows the scan, one pass per token and part of the norm. See `ops.gated_group_norm` for the order of the steps.
#define NORM_KEEP 8   // values of a part that a thread keeps in registers

// G threads per (token, part): a warp for parts of up to 256 elements, a block of 256 threads beyond. A part of up to
// NORM_KEEP * G elements stays in registers and every input is read once, all loads of a thread asked for together;
// longer parts are computed twice.
template <typename T, int G>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ gate, int gate_stride, const T* __restrict__ weight,
                        float eps, T* __restrict__ out, int n_tokens, int width, int n_parts, int n_heads, int gate_kind,
                        int gate_first, const float* __restrict__ nq, const float* __restrict__ floor_in, float floor_add,
                        const float* __restrict__ skip, const T* __restrict__ skip_x, int skip_stride) {
    grid_chain_entry();
    __shared__ float scratch[33];
    const int member = threadIdx.x % G;
    const long long item = (long long)blockIdx.x * (256 / G) + threadIdx.x / G;
    const bool live = item < (long long)n_tokens * n_parts;   // (a warp is live or not as a whole; a block of G = 256 too)
    const int t = live ? (int)(item / n_parts) : 0, part = live ? (int)(item % n_parts) : 0;
    const int part_width = width / n_parts, head_width = width / n_heads, c0 = part * part_width, c_end = c0 + part_width;
    auto gate_of = [&](int c) {
        const float raw = Num<T>::to_f(gate[(size_t)t * gate_stride + c]);
        const float sig = 1.f / (1.f + expf(-raw));
        return gate_kind == 0 ? sig : raw * sig;
    };
    auto value = [&](int c) {
        const int head = c / head_width;
        float z = y[(size_t)t * width + c];
        if (nq) z = z / (fmaxf(fabsf(nq[(size_t)t * n_heads + head]), floor_in[(size_t)t * n_heads + head]) + floor_add);
        if (skip) z = fmaf(skip[head], Num<T>::to_f(skip_x[(size_t)t * skip_stride + c]), z);
        return gate_first ? z * gate_of(c) : z;
    };
    auto total = [&](float v) {
        if (G == 32) return warp_sum(v);
        return block_sum(v, scratch);
    };
    if (G == 32 && !live) return;
    const bool single = part_width <= NORM_KEEP * G;
    float kept[NORM_KEEP], sum = 0.f;
    if (single) {
#pragma unroll
        for (int i = 0; i < NORM_KEEP; ++i) {
            const int c = c0 + member + G * i;
            kept[i] = live && c < c_end ? value(c) : 0.f;
            sum = fmaf(kept[i], kept[i], sum);
        }
    } else if (live) {
        for (int c = c0 + member; c < c_end; c += G) {
            const float z = value(c);
            sum = fmaf(z, z, sum);
        }
    }
    const float inv = rsqrtf(total(sum) / (float)part_width + eps);
    if (!live) return;
    if (single) {
#pragma unroll
        for (int i = 0; i < NORM_KEEP; ++i) {
            const int c = c0 + member + G * i;
            if (c >= c_end) continue;
            float z = kept[i] * inv * Num<T>::to_f(weight[c]);
            if (!gate_first) z *= gate_of(c);
            out[(size_t)t * width + c] = Num<T>::from_f(z);
        }
    } else {
        for (int c = c0 + member; c < c_end; c += G) {
            float z = value(c) * inv * Num<T>::to_f(weight[c]);
            if (!gate_first) z *= gate_of(c);
            out[(size_t)t * width + c] = Num<T>::from_f(z);
        }
    }
}

template <typename T, int G>
static int launch_norm(const float* y, const void* gate, int gate_stride, const void* weight, float eps, void* out, int n_tokens,
                       int width, int n_parts, int n_heads, int gate_kind, int gate_first, const float* nq, const float* floor_in,
                       float floor_add, const float* skip, const void* skip_x, int skip_stride, cudaStream_t stream) {
    const long long items = (long long)n_tokens * n_parts, per_block = 256 / G;
    return (int)launch_pdl(gated_group_norm_kernel<T, G>, dim3((unsigned)((items + per_block - 1) / per_block)), dim3(256), 0, stream,
                           y, (const T*)gate, gate_stride, (const T*)weight, eps, (T*)out, n_tokens, width, n_parts, n_heads,
                           gate_kind, gate_first, nq, floor_in, floor_add, skip, (const T*)skip_x, skip_stride);
}

QF_EXPORT int qf_gated_group_norm(int is_bf16, const float* y, const void* gate, int gate_stride, const void* weight, float eps,
                                  void* out, int n_tokens, int width, int n_parts, int n_heads, int gate_kind, int gate_first,
                                  const float* nq, const float* floor_in, float floor_add, const float* skip, const void* skip_x,
                                  int skip_stride, cudaStream_t stream) {
    if ((long long)n_tokens * n_parts <= 0) return 0;
    if (width % n_parts || width % n_heads) return (int)cudaErrorInvalidValue;
#define QF_NORM_ARGS y, gate, gate_stride, weight, eps, out, n_tokens, width, n_parts, n_heads, gate_kind, gate_first, nq, floor_in, \
                     floor_add, skip, skip_x, skip_stride, stream
    if (width / n_parts <= 32 * NORM_KEEP) return is_bf16 ? launch_norm<bf16, 32>(QF_NORM_ARGS) : launch_norm<float, 32>(QF_NORM_ARGS);
    return is_bf16 ? launch_norm<bf16, 256>(QF_NORM_ARGS) : launch_norm<float, 256>(QF_NORM_ARGS);
#undef QF_NORM_ARGS
}

// ------------------------------------------------------------------------------------------------------------------
// Causal convolution per channel over a sequence's tokens, then silu. A thread takes one (token, channel); what lies
// before the step's first token comes from the sequence's state (its last taps - 1 inputs). A second kernel then moves
// the step's last taps - 1 inputs into the state, a thread per (sequence, channel), reading all it needs before it writes.
// In a step of ONE token per sequence (`single`) a channel's kept inputs have one reader, the thread of that token and
// channel, which then moves them itself: no second kernel.
#define CONV_MAX_TAPS 16

template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ weight,
                                        const float* __restrict__ bias, const int* __restrict__ cu_q,
                                        const int* __restrict__ tok_seq, const int* __restrict__ slots,
                                        float* __restrict__ state, long long slot_stride, long long offset, int taps,
                                        int n_tokens, int channels, T* __restrict__ out, int plain, int single) {
    grid_chain_entry();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_tokens * channels) return;
    const int t = (int)(i / channels), c = (int)(i % channels);
    const int seq = tok_seq[t], at = t - cu_q[seq], slot = slots[seq];
    float* before = slot >= 0 ? state + slot * slot_stride + offset : nullptr;   // [taps - 1][channels]
    float z = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {          // oldest input first: the same order for every cut
        const int back = taps - 1 - j;
        float u = 0.f;
        if (at - back >= 0) u = Num<T>::to_f(x[(size_t)(t - back) * x_stride + c]);
        else if (before) u = before[(size_t)(taps - 1 + at - back) * channels + c];
        z = fmaf(weight[(size_t)c * taps + j], u, z);
        // the input that was `back` tokens back is `back + 1` back for the next token: one row further down
        if (single && before && back >= 1 && back < taps - 1) before[(size_t)(taps - 2 - back) * channels + c] = u;
    }
    if (single && before && taps > 1) before[(size_t)(taps - 2) * channels + c] = Num<T>::to_f(x[(size_t)t * x_stride + c]);
    out[(size_t)t * channels + c] = Num<T>::from_f(plain ? z : z / (1.f + expf(-z)));
}

// The same convolution for long steps: a thread takes 16 bytes of channels and a run of CONV_RUN(TAPS) consecutive tokens, keeps
// the last TAPS - 1 inputs in registers as it walks down the run, and fetches them afresh (from the state, or zeros) where a
// sequence begins inside the run. Every output is the same chain of fused multiply-adds, oldest input first, as in the
// kernel of one thread per (token, channel): the two agree bit for bit.
// tokens of a run: the more taps, the more a longer run saves (taps - 1 inputs are fetched again at the start of every run)
#define CONV_RUN(TAPS) ((TAPS) >= 4 ? 8 : 4)

template <typename T, int TAPS>
__global__ void __launch_bounds__(128)
causal_conv_run_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ weight, const float* __restrict__ bias,
                       const int* __restrict__ cu_q, const int* __restrict__ tok_seq, const int* __restrict__ slots,
                       const float* __restrict__ state, long long slot_stride, long long offset, int n_tokens, int channels,
                       T* __restrict__ out, int plain) {
    constexpr int V = 16 / (int)sizeof(T);
    constexpr int H = TAPS > 1 ? TAPS - 1 : 1;
    grid_chain_entry();
    const int groups = channels / V;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    constexpr int RUN = CONV_RUN(TAPS);
    const int n_runs = (n_tokens + RUN - 1) / RUN;
    if (i >= (long long)n_runs * groups) return;
    const int t0 = (int)(i / groups) * RUN, c0 = (int)(i % groups) * V;
    float w[V][TAPS], b[V], hist[H][V];
#pragma unroll
    for (int v = 0; v < V; ++v) {
        b[v] = bias ? bias[c0 + v] : 0.f;
#pragma unroll
        for (int j = 0; j < TAPS; ++j) w[v][j] = weight[(size_t)(c0 + v) * TAPS + j];
    }
#pragma unroll
    for (int k = 0; k < RUN; ++k) {
        const int t = t0 + k;
        if (t >= n_tokens) break;
        const int seq = tok_seq[t], at = t - cu_q[seq];
        if (TAPS > 1 && (k == 0 || at == 0)) {
            const int slot = slots[seq];
            const float* before = slot >= 0 ? state + slot * slot_stride + offset : nullptr;
#pragma unroll
            for (int r = 0; r < TAPS - 1; ++r) {   // hist[r]: the input TAPS - 1 - r tokens back
                const int back = TAPS - 1 - r;
                if (at - back >= 0) {
                    T in[V];
                    *reinterpret_cast<uint4*>(in) = *reinterpret_cast<const uint4*>(x + (size_t)(t - back) * x_stride + c0);
#pragma unroll
                    for (int v = 0; v < V; ++v) hist[r][v] = Num<T>::to_f(in[v]);
                } else {
#pragma unroll
                    for (int v = 0; v < V; ++v)
                        hist[r][v] = before ? before[(size_t)(TAPS - 1 + at - back) * channels + c0 + v] : 0.f;
                }
            }
        }
        T in[V], res[V];
        *reinterpret_cast<uint4*>(in) = *reinterpret_cast<const uint4*>(x + (size_t)t * x_stride + c0);
#pragma unroll
        for (int v = 0; v < V; ++v) {
            const float u = Num<T>::to_f(in[v]);
            float z = b[v];
#pragma unroll
            for (int r = 0; r < TAPS - 1; ++r) z = fmaf(w[v][r], hist[r][v], z);
            z = fmaf(w[v][TAPS - 1], u, z);
            res[v] = Num<T>::from_f(plain ? z : z / (1.f + expf(-z)));
#pragma unroll
            for (int r = 0; r + 1 < TAPS - 1; ++r) hist[r][v] = hist[r + 1][v];
            if (TAPS > 1) hist[H - 1][v] = u;
        }
        *reinterpret_cast<uint4*>(out + (size_t)t * channels + c0) = *reinterpret_cast<const uint4*>(res);
    }
}

template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ x, int x_stride, const int* __restrict__ cu_q,
                                  const int* __restrict__ slots, int n_seqs, float* __restrict__ state, long long slot_stride,
                                  long long offset, int taps, int channels) {
    grid_chain_entry();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_seqs * channels) return;
    const int seq = (int)(i / channels), c = (int)(i % channels);
    const int slot = slots[seq], begin = cu_q[seq], len = cu_q[seq + 1] - begin;
    if (slot < 0 || len <= 0) return;
    float* kept = state + slot * slot_stride + offset;
    float next[CONV_MAX_TAPS];
    for (int r = 0; r < taps - 1; ++r) {
        const int at = len - (taps - 1) + r;   // index among the step's tokens; negative: still one of the old inputs
        next[r] = at >= 0 ? Num<T>::to_f(x[(size_t)(begin + at) * x_stride + c]) : kept[(size_t)(taps - 1 + at) * channels + c];
    }
    for (int r = 0; r < taps - 1; ++r) kept[(size_t)r * channels + c] = next[r];
}

template <typename T>
static int launch_conv(const void* x, int x_stride, const float* weight, const float* bias, const int* cu_q, const int* tok_seq,
                       const int* slots, int n_seqs, float* state, long long slot_stride, long long offset, int taps,
                       int n_tokens, int channels, void* out, int plain, int single, cudaStream_t stream) {
    const long long total = (long long)n_tokens * channels;
    constexpr int V = 16 / (int)sizeof(T);
    const bool runs = !single && n_tokens >= 32 && (taps == 2 || taps == 3 || taps == 4) && channels % V == 0 &&
                      x_stride % V == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0;
    cudaError_t e;
    if (runs) {
        const int run = CONV_RUN(taps);
        const long long items = (long long)((n_tokens + run - 1) / run) * (channels / V);
        const dim3 grid((unsigned)((items + 127) / 128)), block(128);
#define QF_CONV_RUN(TAPS) launch_pdl(causal_conv_run_kernel<T, TAPS>, grid, block, 0, stream, (const T*)x, x_stride, weight, bias, \
                                     cu_q, tok_seq, slots, (const float*)state, slot_stride, offset, n_tokens, channels, (T*)out, plain)
        e = taps == 2 ? QF_CONV_RUN(2) : taps == 3 ? QF_CONV_RUN(3) : QF_CONV_RUN(4);
#undef QF_CONV_RUN
    } else {
        e = launch_pdl(causal_conv_silu_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                       (const T*)x, x_stride, weight, bias, cu_q, tok_seq, slots, state, slot_stride, offset,
                       taps, n_tokens, channels, (T*)out, plain, single);
    }
    if (e != cudaSuccess || taps <= 1 || single) return (int)e;
    const long long pairs = (long long)n_seqs * channels;
    // launched the ordinary way: it must not start before every block of the convolution has read the old state
    conv_state_kernel<T><<<dim3((unsigned)((pairs + 255) / 256)), dim3(256), 0, stream>>>((const T*)x, x_stride, cu_q, slots, n_seqs,
                                                                                        state, slot_stride, offset, taps, channels);
    return (int)cudaGetLastError();
}

// plain: 1 leaves the activation out (the convolution alone). single: 1 promises that every sequence of the step brings
// exactly one token (n_tokens == n_seqs).
QF_EXPORT int qf_causal_conv(int is_bf16, const void* x, int x_stride, const float* weight, const float* bias,
                             const int* cu_q, const int* tok_seq, const int* slots, int n_seqs, float* state,
                             long long slot_stride, long long offset, int taps, int n_tokens, int channels, void* out, int plain,
                             int single, cudaStream_t stream) {
    if (single && n_tokens != n_seqs) return (int)cudaErrorInvalidValue;
    if (n_tokens <= 0 || channels <= 0) return 0;
    if (taps < 1 || taps > CONV_MAX_TAPS) return (int)cudaErrorInvalidValue;
    return is_bf16 ? launch_conv<bf16>(x, x_stride, weight, bias, cu_q, tok_seq, slots, n_seqs, state, slot_stride, offset, taps,
                                       n_tokens, channels, out, plain, single, stream)
                   : launch_conv<float>(x, x_stride, weight, bias, cu_q, tok_seq, slots, n_seqs, state, slot_stride, offset, taps,
                                        n_tokens, channels, out, plain, single, stream);
}

QF_EXPORT int qf_causal_conv_silu(int is_bf16, const void* x, int x_stride, const float* weight, const float* bias,
                                  const int* cu_q, const int* tok_seq, const int* slots, int n_seqs, float* state,
                                  long long slot_stride, long long offset, int taps, int n_tokens, int channels, void* out,
                                  cudaStream_t stream) {
    return qf_causal_conv(is_bf16, x, x_stride, weight, bias, cu_q, tok_seq, slots, n_seqs, state, slot_stride, offset, taps,
                          n_tokens, channels, out, 0, 0, stream);
}
