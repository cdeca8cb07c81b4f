// A small tiled product on the CUDA cores, shared by the kernels whose weight matrix changes from block to block
// (one matrix per head, one per expert): Y[r, c] = sum_k X[r, k] * W[c, k] for a tile of 32 rows x 64 columns.
//
// 256 threads; a thread owns rows {2 ty, 2 ty + 1} and columns {tx, tx + 16, tx + 32, tx + 48}. Every output is one
// chain of fused multiply-adds over k in ascending order, in 32-bit, whatever T is: the sum depends on nothing
// but the row's values, so a row's result is the same bits wherever it lies in a tile, a step or a batch.
// PAIR computes a second product with another matrix over the same rows (the two halves of a gated unit).
#pragma once
#include "common.cuh"

#define TG_ROWS 32
#define TG_COLS 64
#define TG_K 32
#define TG_THREADS 256

struct TileGemmSmem {
    float x[TG_ROWS][TG_K + 1];
    float w[TG_COLS][TG_K + 1];
    float w2[TG_COLS][TG_K + 1];
};

// x: first row of the tile (rows valid), w / w2: first column's weight row (cols valid). Strides in elements.
// XROW maps a tile row to its row pointer (rows may be scattered).
template <typename T, bool PAIR, typename XROW>
__device__ __forceinline__ void tile_product(XROW xrow, int rows, const T* __restrict__ w, const T* __restrict__ w2, size_t ldw,
                                             int cols, int K, float (&acc)[2][4], float (&acc2)[2][4], TileGemmSmem& s) {
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = acc2[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += TG_K) {
#pragma unroll
        for (int i = 0; i < TG_ROWS * TG_K / TG_THREADS; ++i) {
            const int idx = tid + i * TG_THREADS, r = idx / TG_K, k = idx % TG_K;
            s.x[r][k] = (r < rows && k0 + k < K) ? to_f32(__ldcg(xrow(r) + k0 + k)) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < TG_COLS * TG_K / TG_THREADS; ++i) {
            const int idx = tid + i * TG_THREADS, c = idx / TG_K, k = idx % TG_K;
            const bool ok = c < cols && k0 + k < K;
            s.w[c][k] = ok ? to_f32(w[(size_t)c * ldw + k0 + k]) : 0.f;
            if (PAIR) s.w2[c][k] = ok ? to_f32(w2[(size_t)c * ldw + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TG_K; ++k) {
            const float a0 = s.x[2 * ty][k], a1 = s.x[2 * ty + 1][k];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = s.w[tx + 16 * j][k];
                acc[0][j] = fmaf(a0, b, acc[0][j]);
                acc[1][j] = fmaf(a1, b, acc[1][j]);
                if (PAIR) {
                    const float b2 = s.w2[tx + 16 * j][k];
                    acc2[0][j] = fmaf(a0, b2, acc2[0][j]);
                    acc2[1][j] = fmaf(a1, b2, acc2[1][j]);
                }
            }
        }
        __syncthreads();
    }
}
