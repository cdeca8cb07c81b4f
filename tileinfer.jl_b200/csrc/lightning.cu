// Linear attention with a decay per head ("lightning" attention): a matrix state per (sequence, head) that is carried
// from token to token,
//
//   S_t = a_h S_(t-1) + k_t v_t^T        S [dim, vdim], 32-bit, zero at the start of a sequence
//   o_t = S_t^T q_t                      [vdim]
//
// with q, k, v = act(projection) (act: SiLU or none; the activation is applied, and rounded to T, as the rows are read).
//
//   lightning_scan   the recurrence over the tokens a step brings, from the state the earlier steps left; the new state is
//                    written back. One kernel serves prompts and one-token steps.
//   lightning_out    y = T( o / rms(o) * w * sigmoid(g) ): the RMS norm over all heads' outputs together, in 32-bit, times
//                    the output gate; the input of the output projection.
//
// The scan: the columns of S are independent (column j of S sees v_t[j] only), so a block owns 32 columns of one
// (sequence, head) and walks the sequence's tokens in order; its 8 or 16 warps split the rows of S (warp w owns DP rows in a
// row, read from shared memory four at a time), a lane owns one column, the state lives in registers. Tokens are staged 32 at a time in shared memory; the
// warps' partial sums of o meet there once per 32 tokens. A launch of few blocks (one prompt, few heads) shares the rows of S
// out between two blocks per column block, whose two shares of o are added in global memory. A token's result depends on
// the sequence's earlier tokens alone; the order of its sums depends on the sizes and on whether the launch was shared
// out, so results agree to rounding, not bit for bit, between a prompt alone and the same prompt in a large batch.
// Everything is 32-bit arithmetic; nothing of the state, the decay or o is rounded.
#include "common.cuh"

#define LS_COLS 32
#define LS_TOKENS 32
#define LS_MAX_DIM 512

__device__ __forceinline__ float silu_value(float z) { return z / (1.0f + expf(-z)); }

template <typename T, int DP, bool VECTORS, int LS_PARTS>
__global__ void __launch_bounds__(LS_COLS* LS_PARTS) lightning_scan_kernel(
    float* __restrict__ o, const T* qkv, long long ld, int q_off, int k_off, int v_off, float* state,
    const float* __restrict__ decay, const int* cu_seqlens, const int* seq_slots, int H, int D, int V, int act, int split) {
    extern __shared__ float smem[];
    float* qs = smem;                                   // [LS_TOKENS][D]
    float* ks = qs + LS_TOKENS * D;                     // [LS_TOKENS][D]
    float* vs = ks + LS_TOKENS * D;                     // [LS_TOKENS][LS_COLS]
    float* part = vs + LS_TOKENS * LS_COLS;             // [LS_TOKENS][LS_PARTS][LS_COLS]
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    // With `split` > 1 the rows of S are shared out among that many blocks, whose shares of o are added up in global memory.
    const int col0 = (blockIdx.x / split) * LS_COLS, h = blockIdx.y, b = blockIdx.z;
    const int rows_per = (D + split - 1) / split, row0 = (blockIdx.x % split) * rows_per, row1 = min(D, row0 + rows_per);
    const int col = col0 + lane;
    const float a = decay[h];
    pdl_enter();
    const int t0 = __ldcg(cu_seqlens + b), t1 = __ldcg(cu_seqlens + b + 1);
    const int slot = __ldcg(seq_slots + b);
    float* S = state + ((size_t)slot * H + h) * D * V;
    float s[DP];
#pragma unroll
    for (int i = 0; i < DP; ++i) {
        const int d = row0 + w * DP + i;
        s[i] = (d < row1 && col < V) ? __ldcg(S + (size_t)d * V + col) : 0.f;
    }
    // The rows of a batch of 16 tokens come in 16-byte vectors where the layout allows it, and the next batch's are asked for
    // before this batch's arithmetic, so that their way from memory is hidden behind it.
    constexpr int VEC = 16 / (int)sizeof(T), MAXV = 4;
    const bool wide = VECTORS && D % VEC == 0 && V % VEC == 0;
    const int qk_vecs = D / VEC;                        // vectors in a head's row of q (and of k)
    constexpr int V_VECS = LS_COLS / VEC;               // vectors in the block's 32 columns of v
    uint4 rq[MAXV], rk[MAXV], rv;
    auto fetch = [&](int base, int count) {
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int idx = threadIdx.x + i * (LS_COLS * LS_PARTS);
            if (idx < count * qk_vecs) {
                const T* row = qkv + (size_t)(base + idx / qk_vecs) * ld + (size_t)h * D + (idx % qk_vecs) * VEC;
                rq[i] = __ldcg(reinterpret_cast<const uint4*>(row + q_off));
                rk[i] = __ldcg(reinterpret_cast<const uint4*>(row + k_off));
            }
        }
        const int idx = threadIdx.x;
        if (idx < count * V_VECS && col0 + (idx % V_VECS) * VEC < V)
            rv = __ldcg(reinterpret_cast<const uint4*>(qkv + (size_t)(base + idx / V_VECS) * ld + v_off + (size_t)h * V + col0 + (idx % V_VECS) * VEC));
    };
    auto put = [&](float* dst, const uint4& raw) {
        Vec16<T> v;
        if constexpr (sizeof(T) == 2) v.unpack(raw);
        else { v.v[0] = __uint_as_float(raw.x); v.v[1] = __uint_as_float(raw.y); v.v[2] = __uint_as_float(raw.z); v.v[3] = __uint_as_float(raw.w); }
#pragma unroll
        for (int e = 0; e < VEC; ++e)           // (16-bit rows: the fast exponential and division are far below their rounding)
            dst[e] = !act ? v.v[e] : sizeof(T) == 2 ? rnd<T>(__fdividef(v.v[e], 1.0f + __expf(-v.v[e]))) : silu_value(v.v[e]);
    };
    if (wide && t0 < t1) fetch(t0, min(LS_TOKENS, t1 - t0));
    for (int base = t0; base < t1; base += LS_TOKENS) {
        const int count = min(LS_TOKENS, t1 - base);
        // (No barrier here: every thread has passed the barrier after the last batch's arithmetic, so its rows may be
        // overwritten; the shares of o that slow threads may still be adding up are rewritten only after the next barrier.)
        if (wide) {
#pragma unroll
            for (int i = 0; i < MAXV; ++i) {
                const int idx = threadIdx.x + i * (LS_COLS * LS_PARTS);
                if (idx < count * qk_vecs) {
                    put(qs + (idx / qk_vecs) * D + (idx % qk_vecs) * VEC, rq[i]);
                    put(ks + (idx / qk_vecs) * D + (idx % qk_vecs) * VEC, rk[i]);
                }
            }
            const int idx = threadIdx.x;
            if (idx < count * V_VECS) {
                float* dst = vs + (idx / V_VECS) * LS_COLS + (idx % V_VECS) * VEC;
                if (col0 + (idx % V_VECS) * VEC < V) put(dst, rv);
                else
#pragma unroll
                    for (int e = 0; e < VEC; ++e) dst[e] = 0.f;
            }
            if (base + LS_TOKENS < t1) fetch(base + LS_TOKENS, min(LS_TOKENS, t1 - base - LS_TOKENS));
        } else {
        for (int e = threadIdx.x; e < count * D; e += blockDim.x) {
            const int t = e / D, d = e % D;
            const T* row = qkv + (size_t)(base + t) * ld + (size_t)h * D + d;
            float qv = to_f32(__ldcg(row + q_off)), kv = to_f32(__ldcg(row + k_off));
            if (act) { qv = rnd<T>(silu_value(qv)); kv = rnd<T>(silu_value(kv)); }
            qs[t * D + d] = qv;
            ks[t * D + d] = kv;
        }
        for (int e = threadIdx.x; e < count * LS_COLS; e += blockDim.x) {
            const int t = e / LS_COLS, c = e % LS_COLS;
            float vv = 0.f;
            if (col0 + c < V) {
                vv = to_f32(__ldcg(qkv + (size_t)(base + t) * ld + v_off + (size_t)h * V + col0 + c));
                if (act) vv = rnd<T>(silu_value(vv));
            }
            vs[t * LS_COLS + c] = vv;
        }
        }
        __syncthreads();
        // One token: the state's rows of this warp move on and give their share of o. Four partial sums keep the chain of
        // dependent additions short; the order of a token's sum still depends on the sizes alone.
        auto token = [&](int t) {
            const float vt = vs[t * LS_COLS + lane];
            const float* qt = qs + t * D;
            const float* kt = ks + t * D;
            float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
            if (D % 4 == 0 && rows_per % 4 == 0) {       // (DP is a multiple of 4: four rows' k and q per shared-memory read)
#pragma unroll
                for (int i = 0; i < DP; i += 4) {
                    const int d = row0 + w * DP + i;
                    if (d < row1) {
                        const float4 k4 = *reinterpret_cast<const float4*>(kt + d), q4 = *reinterpret_cast<const float4*>(qt + d);
                        s[i] = fmaf(a, s[i], k4.x * vt); acc0 = fmaf(s[i], q4.x, acc0);
                        s[i + 1] = fmaf(a, s[i + 1], k4.y * vt); acc1 = fmaf(s[i + 1], q4.y, acc1);
                        s[i + 2] = fmaf(a, s[i + 2], k4.z * vt); acc2 = fmaf(s[i + 2], q4.z, acc2);
                        s[i + 3] = fmaf(a, s[i + 3], k4.w * vt); acc3 = fmaf(s[i + 3], q4.w, acc3);
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < DP; ++i) {
                    const int d = row0 + w * DP + i;
                    if (d < row1) {
                        s[i] = fmaf(a, s[i], kt[d] * vt);
                        acc0 = fmaf(s[i], qt[d], acc0);
                    }
                }
            }
            part[(t * LS_PARTS + w) * LS_COLS + lane] = (acc0 + acc1) + (acc2 + acc3);
        };
        if (count == LS_TOKENS) {
#pragma unroll 4
            for (int t = 0; t < LS_TOKENS; ++t) token(t);
        } else {
            for (int t = 0; t < count; ++t) token(t);
        }
        __syncthreads();
        for (int e = threadIdx.x; e < count * LS_COLS; e += blockDim.x) {
            const int t = e / LS_COLS, c = e % LS_COLS;
            if (col0 + c >= V) continue;
            float sum = 0.f;
#pragma unroll
            for (int p = 0; p < LS_PARTS; ++p) sum += part[(t * LS_PARTS + p) * LS_COLS + c];
            float* dst = o + (size_t)(base + t) * H * V + (size_t)h * V + col0 + c;
            if (split > 1) atomicAdd(dst, sum);         // o was zeroed; with two addends the sum does not depend on their order
            else *dst = sum;
        }
    }
#pragma unroll
    for (int i = 0; i < DP; ++i) {
        const int d = row0 + w * DP + i;
        if (d < row1 && col < V) S[(size_t)d * V + col] = s[i];
    }
}

// One token per sequence: the step reads and writes every state once and is bound by that traffic. A block owns 128 columns
// of one (sequence, head): a lane owns four of them (16 bytes of a row), the warps take the rows in turn with several rows'
// loads in flight, and their shares of o meet in shared memory. The arithmetic per element is the scan's.
#define LT_WARPS 8
template <typename T>
__global__ void __launch_bounds__(LT_WARPS * 32) lightning_token_kernel(float* __restrict__ o, const T* qkv, long long ld, int q_off, int k_off,
                                                                        int v_off, float* state, const float* __restrict__ decay,
                                                                        const int* seq_slots, int H, int D, int V, int act) {
    extern __shared__ float smem[];
    float* qs = smem;                                   // [D]
    float* ks = qs + D;                                 // [D]
    float* part = ks + D;                               // [LT_WARPS][128]
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int col = blockIdx.x * 128 + lane * 4, h = blockIdx.y, b = blockIdx.z;
    const float a = decay[h];
    pdl_enter();
    const T* row = qkv + (size_t)b * ld;
    for (int d = threadIdx.x; d < D; d += LT_WARPS * 32) {
        float qv = to_f32(__ldcg(row + q_off + (size_t)h * D + d)), kv = to_f32(__ldcg(row + k_off + (size_t)h * D + d));
        if (act) { qv = rnd<T>(silu_value(qv)); kv = rnd<T>(silu_value(kv)); }
        qs[d] = qv;
        ks[d] = kv;
    }
    float v4[4] = {0.f, 0.f, 0.f, 0.f};
    if (col < V) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            v4[e] = to_f32(__ldcg(row + v_off + (size_t)h * V + col + e));
            if (act) v4[e] = rnd<T>(silu_value(v4[e]));
        }
    }
    __syncthreads();
    float* S = state + ((size_t)__ldcg(seq_slots + b) * H + h) * D * V;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (col < V) {
#pragma unroll 4
        for (int d = w; d < D; d += LT_WARPS) {
            float4 s4 = __ldcg(reinterpret_cast<const float4*>(S + (size_t)d * V + col));
            const float kd = ks[d], qd = qs[d];
            s4.x = fmaf(a, s4.x, kd * v4[0]); s4.y = fmaf(a, s4.y, kd * v4[1]);
            s4.z = fmaf(a, s4.z, kd * v4[2]); s4.w = fmaf(a, s4.w, kd * v4[3]);
            acc[0] = fmaf(s4.x, qd, acc[0]); acc[1] = fmaf(s4.y, qd, acc[1]);
            acc[2] = fmaf(s4.z, qd, acc[2]); acc[3] = fmaf(s4.w, qd, acc[3]);
            *reinterpret_cast<float4*>(S + (size_t)d * V + col) = s4;
        }
    }
    *reinterpret_cast<float4*>(part + w * 128 + lane * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    __syncthreads();
    for (int c = threadIdx.x; c < 128; c += LT_WARPS * 32) {
        if (blockIdx.x * 128 + c >= V) continue;
        float sum = 0.f;
#pragma unroll
        for (int p = 0; p < LT_WARPS; ++p) sum += part[p * 128 + c];
        o[(size_t)b * H * V + (size_t)h * V + blockIdx.x * 128 + c] = sum;
    }
}

// o [n, H * V] float; qkv [n, ld] of T with the heads' queries from column q_off on (H * D of them), keys from k_off, values
// from v_off (H * V); state [slots, H, D, V] float; decay [H] float; cu_seqlens [B + 1], seq_slots [B] (n_tokens in all). act: 1 = SiLU.
extern "C" int ti_lightning_scan(float* o, const void* qkv, long long ld, int q_off, int k_off, int v_off, float* state, const float* decay,
                                 const int* cu_seqlens, const int* seq_slots, int n_tokens, int B, int H, int D, int V, int act, int dtype,
                                 cudaStream_t stream) {
    if (B == 0) return 0;
    TI_REQUIRE(H > 0 && D > 0 && V > 0 && D <= LS_MAX_DIM, "lightning_scan: %d heads of %d x %d (the key size is at most %d)", H, D, V, LS_MAX_DIM);
    TI_REQUIRE(H <= 65535 && B <= 65535, "lightning_scan: %d heads, %d sequences", H, B);
    if (n_tokens == B && V % 4 == 0 && D <= 2048) {      // one token per sequence: the kernel that streams the states
        const size_t smem1 = (size_t)(2 * D + LT_WARPS * 128) * sizeof(float);
        TI_DISPATCH_DTYPE(dtype, (ti_launch(lightning_token_kernel<T>, dim3((V + 127) / 128, H, B), dim3(LT_WARPS * 32), smem1, stream, o, (const T*)qkv, ld,
                                            q_off, k_off, v_off, state, decay, seq_slots, H, D, V, act)));
        return ti_check_launch("lightning_scan");
    }
    // A launch with few blocks (one prompt of a model with few heads) shares the rows of S out between two blocks each.
    const int col_blocks = (V + LS_COLS - 1) / LS_COLS;
    const int split = ((long long)col_blocks * H * B < 100 && D >= 16) ? 2 : 1;
    if (split > 1 && cudaMemsetAsync(o, 0, (size_t)n_tokens * H * V * sizeof(float), stream) != cudaSuccess) return ti_fail("lightning_scan: memset failed");
    const dim3 grid(col_blocks * split, H, B);
    // Few blocks walking long sequences are bound by latency: 16 warps a block then (each with half the rows); many blocks, or
    // one-token steps, which are bound by reading and writing the state, run better with 8.
    const int parts = ((long long)col_blocks * split * H * B <= 160 && n_tokens >= 64 * B) ? 16 : 8;
    const size_t smem = (size_t)(2 * LS_TOKENS * D + LS_TOKENS * LS_COLS + LS_TOKENS * parts * LS_COLS) * sizeof(float);
    const int dp = ((D + split - 1) / split + parts - 1) / parts;
    // 16-byte loads need every row's pieces on 16-byte borders and at most four vectors of q per thread and batch of tokens.
#define LS_LAUNCH2(DP, PARTS)                                                                                                        \
    do {                                                                                                                             \
        constexpr int VEC = 16 / (int)sizeof(T);                                                                                     \
        const bool vectors = aligned16(qkv) && ld % VEC == 0 && q_off % VEC == 0 && k_off % VEC == 0 && v_off % VEC == 0 &&          \
                             LS_TOKENS * (D / VEC) <= 4 * LS_COLS * PARTS;                                                           \
        if (smem > 48 * 1024) {                                                                                                      \
            cudaFuncSetAttribute(lightning_scan_kernel<T, DP, true, PARTS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            cudaFuncSetAttribute(lightning_scan_kernel<T, DP, false, PARTS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        }                                                                                                                            \
        if (vectors)                                                                                                                 \
            ti_launch(lightning_scan_kernel<T, DP, true, PARTS>, grid, dim3(LS_COLS* PARTS), smem, stream, o, (const T*)qkv, ld, q_off, k_off,    \
                      v_off, state, decay, cu_seqlens, seq_slots, H, D, V, act, split);                                              \
        else                                                                                                                         \
            ti_launch(lightning_scan_kernel<T, DP, false, PARTS>, grid, dim3(LS_COLS* PARTS), smem, stream, o, (const T*)qkv, ld, q_off, k_off,   \
                      v_off, state, decay, cu_seqlens, seq_slots, H, D, V, act, split);                                              \
    } while (0)
#define LS_LAUNCH(DP)                        \
    do {                                     \
        if (parts == 16) LS_LAUNCH2(DP, 16); \
        else LS_LAUNCH2(DP, 8);              \
    } while (0)
    TI_DISPATCH_DTYPE(dtype, {
        if (dp <= 4) LS_LAUNCH(4);
        else if (dp <= 8) LS_LAUNCH(8);
        else if (dp <= 16) LS_LAUNCH(16);
        else if (dp <= 32) LS_LAUNCH(32);
        else LS_LAUNCH(64);
    });
#undef LS_LAUNCH2
#undef LS_LAUNCH
    return ti_check_launch("lightning_scan");
}

template <typename T>
__global__ void lightning_out_kernel(T* __restrict__ y, const float* o, const T* g, long long ldg, const T* __restrict__ w, float eps, int size) {
    __shared__ float scratch[33];
    const float* row = o + (size_t)blockIdx.x * size;
    float ss = 0.f;
    pdl_enter();
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = __ldcg(row + i);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)size + eps);
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        float v = __ldcg(row + i) * inv * to_f32(w[i]);
        if (g != nullptr) v = v / (1.0f + expf(-to_f32(__ldcg(g + (size_t)blockIdx.x * ldg + i))));
        y[(size_t)blockIdx.x * size + i] = from_f32<T>(v);
    }
}

// y [n, size] = T(o / rms(o) * w * sigmoid(g)); o [n, size] float, g [n, ldg] of T (null: no gate), w [size].
extern "C" int ti_lightning_out(void* y, const float* o, const void* g, long long ldg, const void* w, float eps, int n, int size, int dtype,
                                cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(size > 0, "lightning_out: size %d", size);
    const int threads = size >= 4096 ? 512 : size >= 1024 ? 256 : 128;
    TI_DISPATCH_DTYPE(dtype, (ti_launch(lightning_out_kernel<T>, dim3(n), dim3(threads), 0, stream, (T*)y, o, (const T*)g, ldg, (const T*)w, eps, size)));
    return ti_check_launch("lightning_out");
}
