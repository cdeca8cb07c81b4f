// One small matrix per head: y[t, h, :] = W[h] x[t, h, :], W[h] stored [out_h, in_h] row-major, heads one after the
// other. Latent attention uses it twice: to carry a head's query into the key/value latent's space (W[h] = the
// head's key up-projection, transposed) and to carry the attended latent back to the head's values (W[h] = the
// head's value up-projection). 32-bit accumulation in ascending k, one rounding on store.
#include "tile_gemm.cuh"

template <typename T>
__global__ void __launch_bounds__(TG_THREADS) head_gemm_kernel(T* __restrict__ y, size_t ldy, const T* x, size_t ldx,
                                                               const T* __restrict__ w, int n, int out_h, int in_h) {
    __shared__ TileGemmSmem s;
    const int row0 = blockIdx.x * TG_ROWS, col0 = blockIdx.y * TG_COLS, h = blockIdx.z;
    const int rows = min(TG_ROWS, n - row0), cols = min(TG_COLS, out_h - col0);
    pdl_enter();
    const T* xb = x + (size_t)row0 * ldx + (size_t)h * in_h;
    auto xrow = [&](int r) { return xb + (size_t)r * ldx; };
    float acc[2][4], unused[2][4];
    tile_product<T, false>(xrow, rows, w + ((size_t)h * out_h + col0) * in_h, (const T*)nullptr, (size_t)in_h, cols, in_h, acc, unused, s);
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = 2 * ty + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = tx + 16 * j;
            if (c < cols) y[(size_t)(row0 + r) * ldy + (size_t)h * out_h + col0 + c] = from_f32<T>(acc[i][j]);
        }
    }
}

extern "C" int ti_head_gemm(void* y, long long ldy, const void* x, long long ldx, const void* w, int n, int heads, int out_h,
                            int in_h, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(n > 0 && heads > 0 && out_h > 0 && in_h > 0 && heads <= 65535, "head_gemm: bad sizes n=%d heads=%d out=%d in=%d", n, heads, out_h, in_h);
    const dim3 grid((n + TG_ROWS - 1) / TG_ROWS, (out_h + TG_COLS - 1) / TG_COLS, heads);
    TI_DISPATCH_DTYPE(dtype, (ti_launch(head_gemm_kernel<T>, grid, dim3(TG_THREADS), 0, stream, (T*)y, (size_t)ldy, (const T*)x,
                                        (size_t)ldx, (const T*)w, n, out_h, in_h)));
    return ti_check_launch("head_gemm");
}
