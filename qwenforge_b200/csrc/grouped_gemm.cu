// Grouped matrix products: many small products C_g = A_g W_g^T in one launch, each group with a weight of its own.
//
// Two ways of saying which rows belong to which group:
//   uniform  every group takes all `rows` rows and its own slice of columns: A_g = A[:, g * a_group_cols : + K],
//            C_g = C[:, g * c_group_cols : + N]. This is a product per attention head (a latent attention's queries
//            taken into the latent space, its latent outputs taken back to value heads).
//   ragged   the rows are sorted by group and cut into tiles of `tile_rows` rows (64 or 128) by a plan on the device
//            (csrc/moe.cu): tile i belongs to group tile_group[i], starts at row tile_row0[i] and ends where the group's
//            rows end (offsets[group + 1]). The grid has a block row for every tile that any routing can have; those
//            beyond n_tiles[0] end at once. This is the experts of a mixture-of-experts feed-forward. With `a_rows`,
//            row r of A is read from A[a_rows[r]]: the sorted rows are gathered on the way in and never stored.
// W_g = W + g * w_group_stride, row-major [N][K] with leading dimension ldw.
//
// Tiles are 64 x 64 (four warps) or, where there are rows enough, 128 x 128 (eight warps, three stages of K in flight).
// bfloat16 runs on the tensor cores (mma.sync m16n8k16, float32 accumulators, cp.async double buffering) when K and all
// strides are multiples of 8 elements and the bases 16-byte aligned; anything else, and float32, runs a plain tiled
// kernel in which every output element is one chain of fused multiply-adds over k = 0 .. K-1 (no TF32). In both, a
// row's result does not depend on which other rows share its tile.
#include "mma.cuh"

struct GroupedArgs {
    const void* a;
    long long lda, a_group_cols;
    const void* w;
    long long w_group_stride, ldw;
    void* c;
    long long ldc, c_group_cols;
    int rows, n, k, n_groups;
    const int* tile_group;   // null: uniform
    const int* tile_row0;
    const int* offsets;
    const int* n_tiles;
    int max_tiles;
    const int* a_rows;       // null: row r of A is row r
    const float* row_scale;  // gated tiles: a factor per row on both halves before the gate (null: 1)
    float gate_limit, gate_alpha;   // gated tiles, gate_limit > 0: the clamped gate min(g, limit) sigmoid(alpha g) (clamp(u) + 1)
    int act;                 // products without a gate: 0 stores the sums; k + 1 stores activate(sum, k) (see common.cuh)
};

// Which group and which rows this block has; false if it has none.
template <int BM>
__device__ __forceinline__ bool grouped_tile(const GroupedArgs& g, int& group, int& row0, int& row_end) {
    if (g.tile_group) {
        if ((int)blockIdx.y >= g.n_tiles[0]) return false;
        group = g.tile_group[blockIdx.y];
        row0 = g.tile_row0[blockIdx.y];
        row_end = min(g.offsets[group + 1], g.rows);
    } else {
        group = blockIdx.z;
        row0 = blockIdx.y * BM;
        row_end = g.rows;
    }
    return row0 < row_end;
}

#define GG_BN 64
#define GG_BK 16

template <typename T>
__global__ void __launch_bounds__(256)
grouped_gemm_plain_kernel(GroupedArgs g) {
    grid_chain_entry();
    __shared__ float a_s[GG_BK][QF_GROUP_BM + 1];
    __shared__ float w_s[GG_BK][GG_BN + 1];
    int group, m0, m_end;
    if (!grouped_tile<QF_GROUP_BM>(g, group, m0, m_end)) return;
    const T* A = (const T*)g.a + (g.tile_group ? 0 : (long long)group * g.a_group_cols);
    const T* W = (const T*)g.w + (long long)group * g.w_group_stride;
    T* C = (T*)g.c + (g.tile_group ? 0 : (long long)group * g.c_group_cols);
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int n0 = blockIdx.x * GG_BN;
    const int N = g.n, K = g.k;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += GG_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + i * 256;
            const int r = idx / GG_BK, k = idx % GG_BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + k;
            a_s[k][r] = (gm < m_end && gk < K) ? Num<T>::to_f(A[(long long)(g.a_rows ? g.a_rows[gm] : gm) * g.lda + gk]) : 0.f;
            w_s[k][r] = (gn < N && gk < K) ? Num<T>::to_f(W[(long long)gn * g.ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GG_BK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = a_s[k][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = w_s[k][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty + 16 * i;
        if (gm >= m_end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx + 16 * j;
            if (gn < N) C[(long long)gm * g.ldc + gn] = Num<T>::from_f(g.act ? activate(acc[i][j], g.act - 1) : acc[i][j]);
        }
    }
}

// bfloat16 on the tensor cores: a block of four warps makes a tile of 64 x 64, warp (wy, wx) its 32 x 32 quarter as
// 2 x 4 tiles of m16n8k16; both operands arrive in slabs of 32 columns of K by 16-byte asynchronous copies, three slabs ahead.
// GATED: W_g = [gate rows | up rows] (n of each) and the tile's 64 weight rows are 32 gate rows and the 32 matching up rows;
// a thread then holds a gate sum and the up sum of the same column, and the block writes 32 columns of
// silu(s g) * (s u), s the row's scale: the gate/up product of an expert and its gate in one kernel.
#define GT_BK 32
#define GT_LD (GT_BK + 8)
#define GT_STAGES 4
template <bool GATED>
__global__ void __launch_bounds__(128)
grouped_gemm_mma_kernel(GroupedArgs g) {
    grid_chain_entry();
    __shared__ __align__(16) bf16 a_s[GT_STAGES][QF_GROUP_BM][GT_LD];
    __shared__ __align__(16) bf16 w_s[GT_STAGES][GG_BN][GT_LD];
    int group, m0, m_end;
    if (!grouped_tile<QF_GROUP_BM>(g, group, m0, m_end)) return;
    const bf16* A = (const bf16*)g.a + (g.tile_group ? 0 : (long long)group * g.a_group_cols);
    const bf16* W = (const bf16*)g.w + (long long)group * g.w_group_stride;
    bf16* C = (bf16*)g.c + (g.tile_group ? 0 : (long long)group * g.c_group_cols);
    const int n0 = blockIdx.x * (GATED ? GG_BN / 2 : GG_BN), N = g.n, K = g.k;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wy = warp >> 1, wx = warp & 1;
    long long a_row[2];   // the two rows of A this thread fetches, through the row map if there is one
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int gm = m0 + ((threadIdx.x + i * 128) >> 2);
        a_row[i] = gm < m_end ? (g.a_rows ? g.a_rows[gm] : gm) : -1;
    }

    auto fetch = [&](int k0, int buf) {
        // 64 rows x 4 chunks of 8 columns for each operand; 128 threads take two chunks of each
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = threadIdx.x + i * 128;
            const int r = idx >> 2, c = (idx & 3) * 8;
            const bool k_ok = k0 + c < K;
            // weight row of tile row r: GATED, rows 0..31 are gate rows n0.., rows 32..63 the up rows of the same columns
            const int col = GATED ? n0 + (r & 31) : n0 + r;
            const long long w_row = GATED ? (r < 32 ? col : (long long)N + col) : col;
            const bool a_ok = k_ok && a_row[i] >= 0, w_ok = k_ok && col < N;
            cp_async_16(&a_s[buf][r][c], a_ok ? A + a_row[i] * g.lda + k0 + c : A, a_ok);
            cp_async_16(&w_s[buf][r][c], w_ok ? W + w_row * g.ldw + k0 + c : W, w_ok);
        }
    };
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
    // A step of a few rows has a handful of blocks that each walk all of K: what bounds them is the chain of fetches, so
    // three slabs are on their way while one is multiplied.
    const int n_slabs = (K + GT_BK - 1) / GT_BK;
    for (int s = 0; s < GT_STAGES - 1; ++s) {
        if (s < n_slabs) fetch(s * GT_BK, s);
        cp_async_commit();
    }
    for (int slab = 0; slab < n_slabs; ++slab) {
        cp_async_wait<GT_STAGES - 2>();
        __syncthreads();   // slab `slab` has arrived for everyone, and everyone is done with the buffer fetched next
        if (slab + GT_STAGES - 1 < n_slabs) fetch((slab + GT_STAGES - 1) * GT_BK, (slab + GT_STAGES - 1) % GT_STAGES);
        cp_async_commit();
        const int buf = slab % GT_STAGES;
#pragma unroll
        for (int ks = 0; ks < GT_BK / 16; ++ks) {
            uint32_t af[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) ldmatrix_x4(af[i], &a_s[buf][32 * wy + 16 * i + (lane & 15)][16 * ks + (lane >> 4) * 8]);
#pragma unroll
            for (int j2 = 0; j2 < 2; ++j2) {  // 16 weight rows per ldmatrix.x4
                uint32_t wf[4];
                // GATED: warp wx has 16 columns: their gate rows (j2 = 0) and their up rows (j2 = 1)
                const int w_base = GATED ? 32 * j2 + 16 * wx : 32 * wx + 16 * j2;
                ldmatrix_x4(wf, &w_s[buf][w_base + (lane >> 4) * 8 + (lane & 7)][16 * ks + ((lane >> 3) & 1) * 8]);
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    mma_bf16_16816(acc[i][2 * j2], af[i], wf[0], wf[1]);
                    mma_bf16_16816(acc[i][2 * j2 + 1], af[i], wf[2], wf[3]);
                }
            }
        }
    }
    cp_async_wait<0>();
    if (GATED) {
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int gm = m0 + 32 * wy + 16 * i + (lane >> 2) + 8 * half;
                if (gm >= m_end) continue;
                const float s = g.row_scale ? g.row_scale[gm] : 1.f;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int gn = n0 + 16 * wx + 8 * j + 2 * (lane & 3);
                    float g0 = s * acc[i][j][2 * half], g1 = s * acc[i][j][2 * half + 1];
                    float u0 = s * acc[i][2 + j][2 * half], u1 = s * acc[i][2 + j][2 * half + 1], slope = 1.f;
                    if (g.gate_limit > 0.f) {   // both halves clamped, the slope inside the sigmoid, one added to the up half
                        const float limit = g.gate_limit;
                        g0 = fminf(g0, limit);
                        g1 = fminf(g1, limit);
                        u0 = fminf(fmaxf(u0, -limit), limit) + 1.0f;
                        u1 = fminf(fmaxf(u1, -limit), limit) + 1.0f;
                        slope = g.gate_alpha;
                    }
                    const float v0 = g0 / (1.0f + expf(-slope * g0)) * u0;
                    const float v1 = g1 / (1.0f + expf(-slope * g1)) * u1;
                    bf16* dst = C + (long long)gm * g.ldc + gn;
                    if (gn + 1 < N && (((uintptr_t)dst) & 3) == 0) *reinterpret_cast<uint32_t*>(dst) = pack_bf16(v0, v1);
                    else {
                        if (gn < N) dst[0] = __float2bfloat16_rn(v0);
                        if (gn + 1 < N) dst[1] = __float2bfloat16_rn(v1);
                    }
                }
            }
        return;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int gm = m0 + 32 * wy + 16 * i + (lane >> 2) + 8 * half;
            if (gm >= m_end) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int gn = n0 + 32 * wx + 8 * j + 2 * (lane & 3);
                bf16* dst = C + (long long)gm * g.ldc + gn;
                float v0 = acc[i][j][2 * half], v1 = acc[i][j][2 * half + 1];
                if (g.act) {
                    v0 = activate(v0, g.act - 1);
                    v1 = activate(v1, g.act - 1);
                }
                if (gn + 1 < N && (((uintptr_t)dst) & 3) == 0) *reinterpret_cast<uint32_t*>(dst) = pack_bf16(v0, v1);
                else {
                    if (gn < N) dst[0] = __float2bfloat16_rn(v0);
                    if (gn + 1 < N) dst[1] = __float2bfloat16_rn(v1);
                }
            }
        }
}

// The large tile: 128 x 128, eight warps as 2 x 4, warp (wy, wx) a quarter of 64 x 32 as 4 x 4 tiles of m16n8k16; slabs of
// 32 columns of K, three in flight.
#define GL_BM 128
#define GL_BN 128
#define GL_STAGES 3
__global__ void __launch_bounds__(256)
grouped_gemm_mma_large_kernel(GroupedArgs g) {
    grid_chain_entry();
    extern __shared__ __align__(16) unsigned char gl_smem[];
    bf16 (*a_s)[GL_BM][GT_LD] = reinterpret_cast<bf16 (*)[GL_BM][GT_LD]>(gl_smem);
    bf16 (*w_s)[GL_BN][GT_LD] = reinterpret_cast<bf16 (*)[GL_BN][GT_LD]>(gl_smem + (size_t)GL_STAGES * GL_BM * GT_LD * sizeof(bf16));
    int group, m0, m_end;
    if (!grouped_tile<GL_BM>(g, group, m0, m_end)) return;
    const bf16* A = (const bf16*)g.a + (g.tile_group ? 0 : (long long)group * g.a_group_cols);
    const bf16* W = (const bf16*)g.w + (long long)group * g.w_group_stride;
    bf16* C = (bf16*)g.c + (g.tile_group ? 0 : (long long)group * g.c_group_cols);
    const int n0 = blockIdx.x * GL_BN, N = g.n, K = g.k;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wy = warp >> 2, wx = warp & 3;
    long long a_row[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int gm = m0 + ((threadIdx.x + i * 256) >> 2);
        a_row[i] = gm < m_end ? (g.a_rows ? g.a_rows[gm] : gm) : -1;
    }
    auto fetch = [&](int k0, int buf) {
        // 128 rows x 4 chunks of 8 columns for each operand; 256 threads take two chunks of each
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = threadIdx.x + i * 256;
            const int r = idx >> 2, c = (idx & 3) * 8;
            const bool k_ok = k0 + c < K;
            const bool a_ok = k_ok && a_row[i] >= 0, w_ok = k_ok && n0 + r < N;
            cp_async_16(&a_s[buf][r][c], a_ok ? A + a_row[i] * g.lda + k0 + c : A, a_ok);
            cp_async_16(&w_s[buf][r][c], w_ok ? W + (long long)(n0 + r) * g.ldw + k0 + c : W, w_ok);
        }
    };
    float acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
    const int n_slabs = (K + GT_BK - 1) / GT_BK;
    for (int s = 0; s < GL_STAGES - 1; ++s) {
        if (s < n_slabs) fetch(s * GT_BK, s);
        cp_async_commit();
    }
    for (int slab = 0; slab < n_slabs; ++slab) {
        cp_async_wait<GL_STAGES - 2>();
        __syncthreads();   // slab `slab` has arrived for everyone, and everyone is done with the buffer fetched next
        if (slab + GL_STAGES - 1 < n_slabs) fetch((slab + GL_STAGES - 1) * GT_BK, (slab + GL_STAGES - 1) % GL_STAGES);
        cp_async_commit();
        const int buf = slab % GL_STAGES;
#pragma unroll
        for (int ks = 0; ks < GT_BK / 16; ++ks) {
            uint32_t af[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) ldmatrix_x4(af[i], &a_s[buf][64 * wy + 16 * i + (lane & 15)][16 * ks + (lane >> 4) * 8]);
#pragma unroll
            for (int j2 = 0; j2 < 2; ++j2) {
                uint32_t wf[4];
                ldmatrix_x4(wf, &w_s[buf][32 * wx + 16 * j2 + (lane >> 4) * 8 + (lane & 7)][16 * ks + ((lane >> 3) & 1) * 8]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    mma_bf16_16816(acc[i][2 * j2], af[i], wf[0], wf[1]);
                    mma_bf16_16816(acc[i][2 * j2 + 1], af[i], wf[2], wf[3]);
                }
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int gm = m0 + 64 * wy + 16 * i + (lane >> 2) + 8 * half;
            if (gm >= m_end) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int gn = n0 + 32 * wx + 8 * j + 2 * (lane & 3);
                bf16* dst = C + (long long)gm * g.ldc + gn;
                float v0 = acc[i][j][2 * half], v1 = acc[i][j][2 * half + 1];
                if (g.act) {
                    v0 = activate(v0, g.act - 1);
                    v1 = activate(v1, g.act - 1);
                }
                if (gn + 1 < N && (((uintptr_t)dst) & 3) == 0) *reinterpret_cast<uint32_t*>(dst) = pack_bf16(v0, v1);
                else {
                    if (gn < N) dst[0] = __float2bfloat16_rn(v0);
                    if (gn + 1 < N) dst[1] = __float2bfloat16_rn(v1);
                }
            }
        }
}

static bool mma_takes(const GroupedArgs& g) {
    const long long strides = g.lda | g.ldw | g.a_group_cols | g.w_group_stride | (long long)g.k;
    return strides % 8 == 0 && ((uintptr_t)g.a | (uintptr_t)g.w) % 16 == 0;
}

// Rows from which uniform groups take the large tile.
#define GL_MIN_ROWS 512

// See the top of the file. tile_group == null: uniform groups over all rows; else the ragged plan (a_group_cols and
// c_group_cols are then not used), whose tiles have `tile_rows` rows: 64, or 128 for the large tile (bfloat16 with aligned
// operands only: see qf_grouped_gemm_large_takes). A, W and C share the activation dtype; a_rows: see the top.
// gate_limit > 0 (gated products only): the clamped form of the gate with this limit and the slope gate_alpha.
// act (products without a gate): 0 stores the sums, k + 1 stores activation k of them (the numbers of common.cuh).
QF_EXPORT int qf_grouped_gemm_act(int is_bf16, const void* a, long long lda, long long a_group_cols, const void* w,
                                  long long w_group_stride, long long ldw, void* c, long long ldc, long long c_group_cols,
                                  int rows, int n, int k, int n_groups, const int* tile_group, const int* tile_row0,
                                  const int* offsets, const int* n_tiles, int max_tiles, int tile_rows, const int* a_rows,
                                  int gated, const float* row_scale, float gate_limit, float gate_alpha, int act,
                                  cudaStream_t stream) {
    if (rows <= 0 || n <= 0 || n_groups <= 0) return 0;
    if (act < 0 || act > 6 || (gated && act)) return (int)cudaErrorInvalidValue;
    GroupedArgs g{a, lda, a_group_cols, w, w_group_stride, ldw, c, ldc, c_group_cols, rows, n, k, n_groups,
                  tile_group, tile_row0, offsets, n_tiles, max_tiles, a_rows, row_scale, gate_limit, gate_alpha, act};
    if (gated) {  // n = columns of the result (half of a group's weight rows); the small tensor-core tile only
        if (!is_bf16 || !mma_takes(g) || (tile_group && tile_rows != QF_GROUP_BM)) return (int)cudaErrorInvalidValue;
        const dim3 grid((n + GG_BN / 2 - 1) / (GG_BN / 2), tile_group ? max_tiles : (rows + QF_GROUP_BM - 1) / QF_GROUP_BM, tile_group ? 1 : n_groups);
        if (grid.y == 0 || grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
        return (int)launch_pdl(grouped_gemm_mma_kernel<true>, grid, dim3(128), 0, stream, g);
    }
    const bool large = tile_group ? tile_rows == GL_BM : (is_bf16 && mma_takes(g) && rows >= GL_MIN_ROWS);
    if (tile_group && tile_rows != GL_BM && tile_rows != QF_GROUP_BM) return (int)cudaErrorInvalidValue;
    if (large) {
        if (!is_bf16 || !mma_takes(g)) return (int)cudaErrorInvalidValue;
        const size_t smem = (size_t)GL_STAGES * (GL_BM + GL_BN) * GT_LD * sizeof(bf16);
        cudaError_t e = cudaFuncSetAttribute(grouped_gemm_mma_large_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        const dim3 grid((n + GL_BN - 1) / GL_BN, tile_group ? max_tiles : (rows + GL_BM - 1) / GL_BM, tile_group ? 1 : n_groups);
        if (grid.y == 0 || grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
        return (int)launch_pdl(grouped_gemm_mma_large_kernel, grid, dim3(256), smem, stream, g);
    }
    const dim3 grid((n + GG_BN - 1) / GG_BN, tile_group ? max_tiles : (rows + QF_GROUP_BM - 1) / QF_GROUP_BM, tile_group ? 1 : n_groups);
    if (grid.y == 0 || grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
    if (is_bf16 && mma_takes(g)) return (int)launch_pdl(grouped_gemm_mma_kernel<false>, grid, dim3(128), 0, stream, g);
    if (is_bf16) return (int)launch_pdl(grouped_gemm_plain_kernel<bf16>, grid, dim3(256), 0, stream, g);
    return (int)launch_pdl(grouped_gemm_plain_kernel<float>, grid, dim3(256), 0, stream, g);
}

QF_EXPORT int qf_grouped_gemm_gate(int is_bf16, const void* a, long long lda, long long a_group_cols, const void* w,
                                   long long w_group_stride, long long ldw, void* c, long long ldc, long long c_group_cols,
                                   int rows, int n, int k, int n_groups, const int* tile_group, const int* tile_row0,
                                   const int* offsets, const int* n_tiles, int max_tiles, int tile_rows, const int* a_rows,
                                   int gated, const float* row_scale, float gate_limit, float gate_alpha, cudaStream_t stream) {
    return qf_grouped_gemm_act(is_bf16, a, lda, a_group_cols, w, w_group_stride, ldw, c, ldc, c_group_cols, rows, n, k, n_groups,
                               tile_group, tile_row0, offsets, n_tiles, max_tiles, tile_rows, a_rows, gated, row_scale, gate_limit,
                               gate_alpha, 0, stream);
}

QF_EXPORT int qf_grouped_gemm(int is_bf16, const void* a, long long lda, long long a_group_cols, const void* w,
                              long long w_group_stride, long long ldw, void* c, long long ldc, long long c_group_cols,
                              int rows, int n, int k, int n_groups, const int* tile_group, const int* tile_row0,
                              const int* offsets, const int* n_tiles, int max_tiles, int tile_rows, const int* a_rows,
                              int gated, const float* row_scale, cudaStream_t stream) {
    return qf_grouped_gemm_gate(is_bf16, a, lda, a_group_cols, w, w_group_stride, ldw, c, ldc, c_group_cols, rows, n, k, n_groups,
                                tile_group, tile_row0, offsets, n_tiles, max_tiles, tile_rows, a_rows, gated, row_scale, 0.f, 0.f,
                                stream);
}

// Whether a ragged product of these operands may use tiles of 128 rows (the plan has to be cut accordingly).
QF_EXPORT int qf_grouped_gemm_large_takes(int is_bf16, const void* a, long long lda, const void* w, long long w_group_stride,
                                          long long ldw, int k) {
    GroupedArgs g{a, lda, 0, w, w_group_stride, ldw, nullptr, 0, 0, 0, 0, k, 0, nullptr, nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0.f, 0.f, 0};
    return is_bf16 && mma_takes(g) ? 1 : 0;
}
