// A tile (64 x 64, or larger) of  C = A W^T  on the tensor cores (mma.sync m16n8k16, bfloat16 in, float accumulate) for
// kernels whose rows are gathered: A's 64 rows and W's 64 rows are each named by a pointer per row (null: a
// row of zeros), both K-contiguous.  Four warps in 2 x 2, a warp owning 32 x 32, or eight in 2 x 4 for 128 x 128; K in steps of 64 through a ring
// of three stages filled by 16-byte asynchronous copies; 16-byte chunks of a row are swizzled by the row so
// that ldmatrix reads without bank conflicts.  K must be a multiple of 8 and every row pointer 16-byte aligned.
//
// Products of bfloat16 numbers are exact in float, so a result differs from float arithmetic on the same
// inputs only in the order and rounding of the float additions.
#pragma once
#include "common.cuh"
#include "attention_mma.cuh"       // cp_async_16, ldmatrix_x4, mma_bf16_16816

namespace vapi {

constexpr int MT_BM = 64, MT_BN = 64, MT_BK = 64, MT_STAGES = 3, MT_THREADS = 128;
constexpr int MT_TILE = MT_BM * MT_BK;                                   // elements of one A (or W) stage
constexpr size_t MT_SMEM = (size_t)2 * MT_STAGES * MT_TILE * sizeof(__nv_bfloat16);     // 48 KB

// The tile for BM x BN with WM x WN warps (a warp owns (BM / WM) x (BN / WN), multiples of 16).
// acc[mi][ni][4]: the warp's rows (warp / WN) * (BM / WM) + mi * 16 + {g, g + 8}, columns
// (warp % WN) * (BN / WN) + ni * 8 + 2t + {0, 1}  (g = lane >> 2, t = lane & 3; elements 0, 1: row g; 2, 3: row g + 8).
// a_rows [BM] / w_rows [BN]: shared arrays of row pointers; `safe`: any valid global address (what a copy of no
// bytes names).  Shared memory: MT_STAGES * (BM + BN) * MT_BK elements.
template <int BM, int BN, int WM, int WN>
struct MmaTile {
    static constexpr int THREADS = WM * WN * 32;
    static constexpr int MI = BM / WM / 16, NI = BN / WN / 8;
    static constexpr size_t SMEM = (size_t)MT_STAGES * (BM + BN) * MT_BK * sizeof(__nv_bfloat16);

    static __device__ __forceinline__ void run(const __nv_bfloat16* const* a_rows, const __nv_bfloat16* const* w_rows, int K,
                                               const __nv_bfloat16* safe, __nv_bfloat16* smem, float (&acc)[MI][NI][4]) {
        __nv_bfloat16* sA = smem;
        __nv_bfloat16* sW = smem + MT_STAGES * BM * MT_BK;
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int wm = warp / WN, wn = warp % WN;
#pragma unroll
        for (int mi = 0; mi < MI; ++mi)
#pragma unroll
            for (int ni = 0; ni < NI; ++ni) acc[mi][ni][0] = acc[mi][ni][1] = acc[mi][ni][2] = acc[mi][ni][3] = 0.f;
        const int nk = (K + MT_BK - 1) / MT_BK;

        auto load = [&](int kt, int stage) {
            const int k0 = kt * MT_BK;
#pragma unroll
            for (int i = 0; i < (BM * 8) / THREADS; ++i) {
                const int idx = threadIdx.x + i * THREADS;
                const int r = idx >> 3, c = idx & 7;
                const int k = k0 + c * 8;
                const __nv_bfloat16* ap = a_rows[r];
                const bool ok = ap && k < K;
                cp_async_16(sA + stage * BM * MT_BK + r * MT_BK + ((c ^ (r & 7)) << 3), ok ? ap + k : safe, ok ? 16 : 0);
            }
#pragma unroll
            for (int i = 0; i < (BN * 8) / THREADS; ++i) {
                const int idx = threadIdx.x + i * THREADS;
                const int r = idx >> 3, c = idx & 7;
                const int k = k0 + c * 8;
                const __nv_bfloat16* wp = w_rows[r];
                const bool ok = wp && k < K;
                cp_async_16(sW + stage * BN * MT_BK + r * MT_BK + ((c ^ (r & 7)) << 3), ok ? wp + k : safe, ok ? 16 : 0);
            }
        };
#pragma unroll
        for (int st = 0; st < MT_STAGES - 1; ++st) {
            if (st < nk) load(st, st);
            cp_async_commit();
        }
        const int mat = lane >> 3, rin = lane & 7;
        for (int kt = 0; kt < nk; ++kt) {
            cp_async_wait<MT_STAGES - 2>();
            __syncthreads();
            if (kt + MT_STAGES - 1 < nk) load(kt + MT_STAGES - 1, (kt + MT_STAGES - 1) % MT_STAGES);
            cp_async_commit();
            const __nv_bfloat16* as = sA + (kt % MT_STAGES) * BM * MT_BK;
            const __nv_bfloat16* ws = sW + (kt % MT_STAGES) * BN * MT_BK;
#pragma unroll
            for (int kk = 0; kk < MT_BK / 16; ++kk) {
                unsigned af[MI][4];
#pragma unroll
                for (int mi = 0; mi < MI; ++mi) {
                    const int row = wm * (BM / WM) + mi * 16 + (mat & 1) * 8 + rin;
                    const int ch = kk * 2 + (mat >> 1);
                    ldmatrix_x4(af[mi][0], af[mi][1], af[mi][2], af[mi][3], as + row * MT_BK + ((ch ^ (row & 7)) << 3));
                }
#pragma unroll
                for (int nj = 0; nj < NI / 2; ++nj) {
                    const int row = wn * (BN / WN) + nj * 16 + (mat >> 1) * 8 + rin;
                    const int ch = kk * 2 + (mat & 1);
                    unsigned r0, r1, r2, r3;
                    ldmatrix_x4(r0, r1, r2, r3, ws + row * MT_BK + ((ch ^ (row & 7)) << 3));
#pragma unroll
                    for (int mi = 0; mi < MI; ++mi) {
                        mma_bf16_16816(acc[mi][2 * nj], af[mi], r0, r1);
                        mma_bf16_16816(acc[mi][2 * nj + 1], af[mi], r2, r3);
                    }
                }
            }
        }
        cp_async_wait<0>();
        __syncthreads();               // the stages may be reused by the caller's epilogue
    }
};

// The 64 x 64 tile of four warps (2 x 2).
__device__ __forceinline__ void mma_tile_64x64(const __nv_bfloat16* const* a_rows, const __nv_bfloat16* const* w_rows, int K,
                                               const __nv_bfloat16* safe, __nv_bfloat16* smem, float (&acc)[2][4][4]) {
    MmaTile<64, 64, 2, 2>::run(a_rows, w_rows, K, safe, smem, acc);
}

}  // namespace vapi
