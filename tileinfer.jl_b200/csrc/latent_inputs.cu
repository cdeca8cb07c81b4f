// Inputs of latent attention: the two down-projected latents of a token, each RMS-normed in 32-bit with a plain
// weight; the query latent goes to a dense buffer, the key/value latent to the token's place in the paged pool
// (one "head" of kv_rank elements per position: pool[slot * kv_rank + i], slot = page * page_size + offset).
//
//   cq = T(a / rms(a) * wq),  a = row[0 : q_rank]
//   c  = T(b / rms(b) * wkv), b = row[q_rank : q_rank + kv_rank]
//
// The row is the fused down projection's output [n, q_rank + kv_rank] in T, or its 32-bit partial sums
// [s, n, q_rank + kv_rank] (a product cut over k), added in split order. One block per token.
#include "common.cuh"

#define LI_THREADS 128

template <typename T>
__global__ void latent_inputs_kernel(const T* rows, size_t row_stride, const float* partials, int n_partials, size_t partial_stride,
                                     T* __restrict__ cq, T* pool, const T* __restrict__ wq, const T* __restrict__ wkv, float eps,
                                     const int* slots, int q_rank, int kv_rank) {
    extern __shared__ float row[];             // [q_rank + kv_rank]
    __shared__ float scratch[33];
    const int t = blockIdx.x, size = q_rank + kv_rank;
    pdl_enter();
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < size; i += LI_THREADS) {
        float v;
        if (partials != nullptr) {
            const float* p = partials + (size_t)t * size + i;
            v = __ldcg(p);
            for (int s = 1; s < n_partials; ++s) v += __ldcg(p + (size_t)s * partial_stride);
        } else {
            v = to_f32(__ldcg(rows + (size_t)t * row_stride + i));
        }
        row[i] = v;
        if (i < q_rank) sq = fmaf(v, v, sq);
        else sk = fmaf(v, v, sk);
    }
    sq = block_sum(sq, scratch);
    sk = block_sum(sk, scratch);
    const float iq = 1.0f / sqrtf(sq / (float)q_rank + eps), ik = 1.0f / sqrtf(sk / (float)kv_rank + eps);
    const size_t slot = (size_t)__ldcg(slots + t);
    for (int i = threadIdx.x; i < size; i += LI_THREADS) {
        if (i < q_rank) cq[(size_t)t * q_rank + i] = from_f32<T>(row[i] * iq * to_f32(wq[i]));
        else pool[slot * kv_rank + (i - q_rank)] = from_f32<T>(row[i] * ik * to_f32(wkv[i - q_rank]));
    }
}

extern "C" int ti_latent_inputs(const void* rows, long long row_stride, const float* partials, int n_partials, long long partial_stride,
                                void* cq, void* pool, const void* wq, const void* wkv, float eps, const int* slots, int n_tokens,
                                int q_rank, int kv_rank, int dtype, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    TI_REQUIRE(q_rank > 0 && kv_rank > 0 && q_rank + kv_rank <= 12000, "latent_inputs: ranks %d and %d", q_rank, kv_rank);
    TI_REQUIRE((rows != nullptr) != (partials != nullptr), "latent_inputs: give rows or partial sums, not both");
    const size_t smem = (size_t)(q_rank + kv_rank) * sizeof(float);
    TI_DISPATCH_DTYPE(dtype, (ti_launch(latent_inputs_kernel<T>, dim3(n_tokens), dim3(LI_THREADS), smem, stream, (const T*)rows,
                                        (size_t)row_stride, partials, n_partials, (size_t)partial_stride, (T*)cq, (T*)pool, (const T*)wq,
                                        (const T*)wkv, eps, slots, q_rank, kv_rank)));
    return ti_check_launch("latent_inputs");
}
