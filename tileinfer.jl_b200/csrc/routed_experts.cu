// A routed feed-forward: every token goes through `top` of `experts` small gated units, chosen by a router.
//
//   router_topk     z = Wr h in 32-bit (one warp per expert and token, lanes stride over the width), score = sigmoid(z);
//                   the `top` largest (ties to the smaller index) -> ids [n, top], scores [n, top]
//   router_select   the same choice for routers with more rules: softmax or sigmoid scores, a correction added for the choice only,
//                   experts in groups of which only the best stay, weights divided by their sum, pass-through choices, a gate
//                   for the units that every token takes
//   expert_plan     the (token, choice) pairs grouped by expert: a row for every pair in expert order, every expert's rows
//                   padded to whole tiles, and the expert of every tile; one block, counts in shared memory
//   expert_gather   xs[row of the pair] = T(score * h[token]) (the score scales an expert's INPUT) or T(h[token]); padding rows
//                   are left as they are (a row's results depend on that row alone, and nobody reads a padding row's)
//   grouped_gemm    for every tile: y[row, :] = W[expert] xs[row, :] on the CUDA cores (the 32-bit path, and sizes the
//                   tensor-core kernel refuses; csrc/gemm_tcgen05.cu has the tensor-core form); as a gated unit W[expert]
//                   holds gate rows then up rows and y = a * sigmoid(slope * a) * (b + shift), a = min(gate, limit),
//                   b = clamp(up, -limit, limit)
//   expert_combine  out[token] = sum over the token's choices, in choice order, of y[row(token, choice)] (times the score
//                   where it scales the OUTPUT) + a shared row, in 32-bit, rounded once (where the score scales the INPUT the
//                   stream's update adds the rows up itself: csrc/stream32.cu)
//
// Nothing here reads a count on the host: grids are sized by upper bounds and blocks beyond the device-side
// counts leave at once, so a step with a routed feed-forward can be captured in a CUDA graph.
// Which row a pair gets inside its expert's range depends on the order in which threads arrive; a row's values do
// not (every row of a product is computed alone, in ascending k), so results are the same bits from run to run.
#include "tile_gemm.cuh"

#define RT_THREADS 128
#define RT_MAX_EXPERTS 1024

template <typename T>
__global__ void router_topk_kernel(const T* h, const T* __restrict__ wr, const float* logits, int width, int experts, int top,
                                   int always, int* __restrict__ ids, float* __restrict__ scores) {
    __shared__ float z[RT_MAX_EXPERTS];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_enter();
    if (logits != nullptr) {                               // a product kernel has left the 32-bit sums
        for (int e = threadIdx.x; e < experts; e += RT_THREADS) z[e] = __ldcg(logits + (size_t)t * experts + e);
    } else {
        const T* row = h + (size_t)t * width;
        for (int e = warp; e < experts; e += RT_THREADS / 32) {
            const T* w = wr + (size_t)e * width;
            float a = 0.f;
            for (int i = lane; i < width; i += 32) a = fmaf(to_f32(__ldcg(row + i)), to_f32(w[i]), a);
            a = warp_sum(a);
            if (lane == 0) z[e] = a;
        }
    }
    __syncthreads();
    if (warp == 0) {
        for (int j = 0; j < top; ++j) {
            float best = -INFINITY;
            int arg = 0x7fffffff;
            for (int e = lane; e < experts; e += 32)
                if (z[e] > best) { best = z[e]; arg = e; }           // ascending e: the first of equals stays
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
                if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
            }
            if (arg >= experts) arg = j;                            // only if every logit left is NaN
            if (lane == 0) {
                ids[(size_t)t * (top + always) + j] = arg;
                scores[(size_t)t * (top + always) + j] = 1.0f / (1.0f + expf(-best));
                z[arg] = -INFINITY;
            }
            __syncwarp();
        }
        // Units that every token goes through follow the chosen ones, numbered after the routed experts, with score one.
        for (int a = lane; a < always; a += 32) {
            ids[(size_t)t * (top + always) + top + a] = experts + a;
            scores[(size_t)t * (top + always) + top + a] = 1.0f;
        }
    }
}

// `logits` [n, experts]: the router's 32-bit sums if a product kernel has computed them (h and wr are then not read), else null.
// `always`: units after the routed experts that every token takes besides (ids experts .. experts + always - 1, score 1);
// ids and scores are [n, top + always].
extern "C" int ti_router_topk(const void* h, const void* wr, const float* logits, int n, int width, int experts, int top, int always,
                              int* ids, float* scores, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(experts >= 1 && experts <= RT_MAX_EXPERTS && top >= 1 && top <= experts && always >= 0, "router_topk: top %d of %d experts", top, experts);
    TI_DISPATCH_DTYPE(dtype, (ti_launch(router_topk_kernel<T>, dim3(n), dim3(RT_THREADS), 0, stream, (const T*)h, (const T*)wr, logits, width,
                                        experts, top, always, ids, scores)));
    return ti_check_launch("router_topk");
}

// A router with more rules. z [n, ldz] holds the 32-bit logits of `total` = experts + pass choices (and, with a gate, one more
// column: the gate's logit); without z the kernel computes them from h and wr (rows in that order). Per token:
//   s = softmax(z[0 .. total)) (or sigmoid of each), c = s + correction (the CHOICE score; correction may be null);
//   the choices form `groups` equal groups of neighbours, a group's score is its largest c, only the `keep` best groups stay
//   (ties to the smaller index); of those the `top` largest c are chosen (ties to the smaller index);
//   weight = s of the chosen, divided by (their sum + 1e-20) with `renormalize`.
// ids [n, top + always]: the chosen expert, or -1 for a pass choice (the last `total - experts`: their output is the input
// itself), whose weights are summed into pass_weight[n]; then `always` units numbered from `experts` on with the weight
// sigmoid(gate logit), or 1 without a gate.
template <typename T>
__global__ void router_select_kernel(const T* h, const T* __restrict__ wr, const float* z_in, long long ldz, int width, int experts, int total,
                                     int softmax, const float* __restrict__ correction, int groups, int keep, int top, int renormalize,
                                     int always, int gate, int* __restrict__ ids, float* __restrict__ scores, float* __restrict__ pass_weight) {
    __shared__ float z[RT_MAX_EXPERTS + 1], c[RT_MAX_EXPERTS], gs[RT_MAX_EXPERTS];
    __shared__ float scratch[33];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int columns = total + (gate ? 1 : 0);
    pdl_enter();
    if (z_in != nullptr) {
        for (int e = threadIdx.x; e < columns; e += RT_THREADS) z[e] = __ldcg(z_in + (size_t)t * ldz + e);
    } else {
        const T* row = h + (size_t)t * width;
        for (int e = warp; e < columns; e += RT_THREADS / 32) {
            const T* w = wr + (size_t)e * width;
            float a = 0.f;
            for (int i = lane; i < width; i += 32) a = fmaf(to_f32(__ldcg(row + i)), to_f32(w[i]), a);
            a = warp_sum(a);
            if (lane == 0) z[e] = a;
        }
    }
    __syncthreads();
    if (softmax) {
        float m = -INFINITY;
        for (int e = threadIdx.x; e < total; e += RT_THREADS) m = fmaxf(m, z[e]);
        m = block_max(m, scratch);
        float sum = 0.f;
        for (int e = threadIdx.x; e < total; e += RT_THREADS) sum += expf(z[e] - m);
        sum = block_sum(sum, scratch);
        for (int e = threadIdx.x; e < total; e += RT_THREADS) z[e] = expf(z[e] - m) / sum;
    } else {
        for (int e = threadIdx.x; e < total; e += RT_THREADS) z[e] = 1.0f / (1.0f + expf(-z[e]));
    }
    __syncthreads();
    for (int e = threadIdx.x; e < total; e += RT_THREADS) c[e] = z[e] + (correction != nullptr ? correction[e] : 0.f);
    __syncthreads();
    const int per = total / groups;
    if (keep < groups) {
        for (int g = threadIdx.x; g < groups; g += RT_THREADS) {
            float best = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, c[e]);
            gs[g] = best;
        }
        __syncthreads();
        // A group stays if fewer than `keep` groups come before it (a larger score, or an equal one with a smaller index).
        for (int g = threadIdx.x; g < groups; g += RT_THREADS) {
            int before = 0;
            for (int o = 0; o < groups; ++o) before += (gs[o] > gs[g] || (gs[o] == gs[g] && o < g)) ? 1 : 0;
            if (before >= keep)
                for (int e = g * per; e < (g + 1) * per; ++e) c[e] = -INFINITY;
        }
        __syncthreads();
    }
    if (warp == 0) {
        float wsum = 0.f;
        const size_t out = (size_t)t * (top + always);
        for (int j = 0; j < top; ++j) {
            float best = -INFINITY;
            int arg = 0x7fffffff;
            for (int e = lane; e < total; e += 32)
                if (c[e] > best) { best = c[e]; arg = e; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
                if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
            }
            if (arg >= total) arg = j;                              // only if nothing comparable is left (NaN)
            if (lane == 0) {
                ids[out + j] = arg;
                scores[out + j] = z[arg];
                c[arg] = -INFINITY;
            }
            wsum += z[arg];
            __syncwarp();
        }
        if (lane == 0) {
            const float div = renormalize ? wsum + 1e-20f : 1.0f;
            float pass = 0.f;
            for (int j = 0; j < top; ++j) {
                const float wgt = scores[out + j] / div;
                scores[out + j] = wgt;
                if (ids[out + j] >= experts) { pass += wgt; ids[out + j] = -1; }
            }
            if (pass_weight != nullptr) pass_weight[t] = pass;
            const float gw = gate ? 1.0f / (1.0f + expf(-z[total])) : 1.0f;
            for (int a = 0; a < always; ++a) {
                ids[out + top + a] = experts + a;
                scores[out + top + a] = gw;
            }
        }
    }
}

extern "C" int ti_router_select(const void* h, const void* wr, const float* z, long long ldz, int n, int width, int experts, int total, int softmax,
                                const float* correction, int groups, int keep, int top, int renormalize, int always, int gate, int* ids,
                                float* scores, float* pass_weight, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(experts >= 0 && total >= experts && total >= 1 && total <= RT_MAX_EXPERTS && top >= 1 && top <= total && always >= 0,
               "router_select: top %d of %d choices (%d experts)", top, total, experts);
    TI_REQUIRE(groups >= 1 && total % groups == 0 && keep >= 1 && keep <= groups && keep * (total / groups) >= top,
               "router_select: %d of %d groups over %d choices for top %d", keep, groups, total, top);
    TI_REQUIRE(total == experts || pass_weight != nullptr, "router_select: pass choices need their weights' output");
    TI_DISPATCH_DTYPE(dtype, (ti_launch(router_select_kernel<T>, dim3(n), dim3(RT_THREADS), 0, stream, (const T*)h, (const T*)wr, z, ldz, width, experts,
                                        total, softmax, correction, groups, keep, top, renormalize, always, gate, ids, scores, pass_weight)));
    return ti_check_launch("router_select");
}

// The plan of a step: the pairs grouped by expert, every expert's rows padded to whole tiles of `tile` rows, so that a
// tile holds rows of one expert only (tensor-core kernels then treat a tile like any other; nobody reads the results of
// padding rows). plan[0] = tiles in use, plan[1 + t] = the expert of tile t. pair_row[pair] = the pair's
// row; row_pair[row] = the row's pair, or -1 for padding, for all `capacity` rows.
__global__ void expert_plan_kernel(const int* ids, int pairs, int experts, int tile, int capacity, int* __restrict__ pair_row,
                                   int* __restrict__ row_pair, int* __restrict__ plan) {
    __shared__ int count[RT_MAX_EXPERTS], first[RT_MAX_EXPERTS];
    pdl_enter();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    for (int r = threadIdx.x; r < capacity; r += blockDim.x) row_pair[r] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = __ldcg(ids + p);
        if (e >= 0) atomicAdd(&count[e], 1);             // a negative id: a choice that needs no unit's matrices
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int tiles = 0;
        for (int e = 0; e < experts; ++e) {
            first[e] = tiles * tile;
            for (int r = 0; r < count[e]; r += tile) plan[1 + tiles++] = e;
            count[e] = 0;
        }
        plan[0] = tiles;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = __ldcg(ids + p);
        if (e < 0) { pair_row[p] = -1; continue; }
        const int row = first[e] + atomicAdd(&count[e], 1);
        pair_row[p] = row;
        row_pair[row] = p;
    }
}

// The most tiles of `tile` rows that `pairs` pairs over `experts` experts can take: every tile holds at least one pair, and
// at most one tile per expert is not full.
extern "C" int ti_expert_plan_max_tiles(int pairs, int experts, int tile) {
    const int by_rows = pairs / tile + experts;
    return pairs < by_rows ? pairs : by_rows;
}

extern "C" int ti_expert_plan(const int* ids, int pairs, int experts, int tile, int capacity, int* pair_row, int* row_pair, int* plan,
                              cudaStream_t stream) {
    if (pairs == 0) return 0;
    TI_REQUIRE(experts >= 1 && experts <= RT_MAX_EXPERTS, "expert_plan: %d experts", experts);
    TI_REQUIRE(tile >= TG_ROWS && tile % TG_ROWS == 0 && capacity == ti_expert_plan_max_tiles(pairs, experts, tile) * tile,
               "expert_plan: tiles of %d rows, capacity %d", tile, capacity);
    ti_launch(expert_plan_kernel, dim3(1), dim3(pairs >= 1024 ? 1024 : 256), 0, stream, ids, pairs, experts, tile, capacity, pair_row,
              row_pair, plan);
    return ti_check_launch("expert_plan");
}

// One row of xs for a pair: xs[pair_row[p]] = T(score * h[token]) (or T(h[token])). Padding rows are left as they are:
// a row's results depend on that row alone, and nobody reads a padding row's.
template <typename T>
__device__ __forceinline__ void gather_pair_row(T* __restrict__ xs, const T* h, int row, int p, float s, int per_token, int width,
                                                int first_thread, int threads) {
    const T* src = h + (size_t)(p / per_token) * width;
    T* dst = xs + (size_t)row * width;
    constexpr int N = Vec16<T>::N;
    if (width % N == 0 && ((((uintptr_t)src) | ((uintptr_t)dst)) & 15) == 0) {          // 16 bytes at a time; the same values
        for (int i = first_thread * N; i < width; i += threads * N) {
            Vec16<T> v;
            v.load_cg(src + i);
#pragma unroll
            for (int e = 0; e < N; ++e) v.v[e] = s * v.v[e];
            v.store(dst + i);
        }
        return;
    }
    for (int i = first_thread; i < width; i += threads) dst[i] = from_f32<T>(s * to_f32(__ldcg(src + i)));
}

template <typename T>
__global__ void expert_gather_kernel(T* __restrict__ xs, const T* h, const int* pair_row, const float* scores, int per_token, int width,
                                     int scale_input) {
    const int p = blockIdx.x;
    pdl_enter();
    if (__ldcg(pair_row + p) < 0) return;                  // a pair without a row (see expert_plan)
    gather_pair_row(xs, h, __ldcg(pair_row + p), p, scale_input ? __ldcg(scores + p) : 1.0f, per_token, width, (int)threadIdx.x, (int)blockDim.x);
}

extern "C" int ti_expert_gather(void* xs, const void* h, const int* pair_row, const float* scores, int pairs, int per_token, int width,
                                int scale_input, int dtype, cudaStream_t stream) {
    if (pairs == 0) return 0;
    TI_DISPATCH_DTYPE(dtype, (ti_launch(expert_gather_kernel<T>, dim3(pairs), dim3(width >= 1024 ? 256 : 128), 0, stream, (T*)xs, (const T*)h,
                                        pair_row, scores, per_token, width, scale_input)));
    return ti_check_launch("expert_gather");
}

// The grouped product on the CUDA cores: block (x, y) computes rows [32 x, 32 x + 32) x columns [64 y, 64 y + 64) with the
// matrix of the plan's tile that holds those rows.
template <typename T, bool GATED>
__global__ void __launch_bounds__(TG_THREADS) grouped_gemm_kernel(T* __restrict__ y, const T* x, const T* __restrict__ w, const int* plan,
                                                                  int tile, int out, int in, const float* __restrict__ limits, float slope,
                                                                  float shift) {
    __shared__ TileGemmSmem s;
    pdl_enter();
    const int row0 = blockIdx.x * TG_ROWS, t = row0 / tile;
    if (t >= __ldcg(plan)) return;
    const int e = __ldcg(plan + 1 + t), rows = TG_ROWS;
    const float limit = GATED ? limits[e] : 0.f;
    const int col0 = blockIdx.y * TG_COLS, cols = min(TG_COLS, out - col0);
    const T* xb = x + (size_t)row0 * in;
    auto xrow = [&](int r) { return xb + (size_t)r * in; };
    // A gated unit's matrix holds `out` gate rows and then `out` up rows.
    const T* we = w + (size_t)e * (GATED ? 2 : 1) * out * in + (size_t)col0 * in;
    float acc[2][4], acc2[2][4];
    tile_product<T, GATED>(xrow, rows, we, we + (size_t)out * in, (size_t)in, cols, in, acc, acc2, s);
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = 2 * ty + i;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = tx + 16 * j;
            if (c >= cols) continue;
            float v = acc[i][j];
            if (GATED) {
                const float a = fminf(rnd<T>(v), limit);
                const float b = fminf(fmaxf(rnd<T>(acc2[i][j]), -limit), limit);
                v = a / (1.0f + expf(-slope * a)) * (b + shift);
            }
            y[(size_t)(row0 + r) * out + col0 + c] = from_f32<T>(v);
        }
    }
}

// `limits` [matrices]: every unit's clamp (gated only).
extern "C" int ti_grouped_gemm(void* y, const void* x, const void* w, const int* plan, int rows, int tile, int out, int in,
                               int gated, const float* limits, float slope, float shift, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    TI_REQUIRE(!gated || limits != nullptr, "grouped_gemm: a gated unit needs its limits");
    TI_REQUIRE(out > 0 && in > 0 && tile % TG_ROWS == 0 && rows % tile == 0, "grouped_gemm: bad sizes out=%d in=%d rows=%d tile=%d", out, in, rows, tile);
    const dim3 grid(rows / TG_ROWS, (out + TG_COLS - 1) / TG_COLS);
    TI_DISPATCH_DTYPE(dtype, {
        if (gated) ti_launch(grouped_gemm_kernel<T, true>, grid, dim3(TG_THREADS), 0, stream, (T*)y, (const T*)x, (const T*)w, plan, tile, out, in, limits, slope, shift);
        else ti_launch(grouped_gemm_kernel<T, false>, grid, dim3(TG_THREADS), 0, stream, (T*)y, (const T*)x, (const T*)w, plan, tile, out, in, limits, slope, shift);
    });
    return ti_check_launch("grouped_gemm");
}

template <typename T>
__global__ void expert_combine_kernel(T* __restrict__ out, const T* y, const int* pair_row, const float* scores, const T* shared,
                                      const T* h, const float* pass_weight, int top, int width, int scale_output) {
    const int t = blockIdx.x;
    pdl_enter();
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float a = 0.f;
        for (int j = 0; j < top; ++j) {
            const int p = t * top + j;
            const int row = __ldcg(pair_row + p);
            if (row < 0) continue;                           // a pair without a row: its share comes with pass_weight
            const float v = to_f32(__ldcg(y + (size_t)row * width + i));
            a += scale_output ? __ldcg(scores + p) * v : v;
        }
        if (shared != nullptr) a += to_f32(__ldcg(shared + (size_t)t * width + i));
        if (pass_weight != nullptr) a = fmaf(__ldcg(pass_weight + t), to_f32(__ldcg(h + (size_t)t * width + i)), a);
        out[(size_t)t * width + i] = from_f32<T>(a);
    }
}

// The same with 16 bytes of outputs per thread (the sums in the same order).
template <typename T>
__global__ void expert_combine_vec_kernel(T* __restrict__ out, const T* y, const int* pair_row, const float* scores, const T* shared,
                                          const T* h, const float* pass_weight, int top, int width, int scale_output) {
    constexpr int N = Vec16<T>::N;
    const int t = blockIdx.x;
    pdl_enter();
    for (int i = threadIdx.x * N; i < width; i += blockDim.x * N) {
        float a[N];
#pragma unroll
        for (int e = 0; e < N; ++e) a[e] = 0.f;
        for (int j = 0; j < top; ++j) {
            const int p = t * top + j;
            const int row = __ldcg(pair_row + p);
            if (row < 0) continue;
            const float w = scale_output ? __ldcg(scores + p) : 1.0f;
            Vec16<T> v;
            v.load_cg(y + (size_t)row * width + i);
#pragma unroll
            for (int e = 0; e < N; ++e) a[e] += scale_output ? w * v.v[e] : v.v[e];
        }
        Vec16<T> v;
        if (shared != nullptr) {
            v.load_cg(shared + (size_t)t * width + i);
#pragma unroll
            for (int e = 0; e < N; ++e) a[e] += v.v[e];
        }
        if (pass_weight != nullptr) {
            const float w = __ldcg(pass_weight + t);
            v.load_cg(h + (size_t)t * width + i);
#pragma unroll
            for (int e = 0; e < N; ++e) a[e] = fmaf(w, v.v[e], a[e]);
        }
#pragma unroll
        for (int e = 0; e < N; ++e) v.v[e] = a[e];
        v.store(out + (size_t)t * width + i);
    }
}

// `pass_weight` [n] with `h` [n, width] (both or neither): pass_weight[t] * h[t] is added, the share of choices that hand their
// input through unchanged.
extern "C" int ti_expert_combine(void* out, const void* y, const int* pair_row, const float* scores, const void* shared, const void* h,
                                 const float* pass_weight, int n, int top, int width, int scale_output, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE((h != nullptr) == (pass_weight != nullptr), "expert_combine: the passed-through share needs both its weights and the input");
    TI_DISPATCH_DTYPE(dtype, {
        constexpr int N = Vec16<T>::N;
        if (width % N == 0 && aligned16(out) && aligned16(y) && aligned16(shared) && aligned16(h))
            ti_launch(expert_combine_vec_kernel<T>, dim3(n), dim3(width >= 2048 ? 256 : 128), 0, stream, (T*)out, (const T*)y, pair_row, scores,
                      (const T*)shared, (const T*)h, pass_weight, top, width, scale_output);
        else
            ti_launch(expert_combine_kernel<T>, dim3(n), dim3(width >= 1024 ? 256 : 128), 0, stream, (T*)out, (const T*)y, pair_row, scores,
                      (const T*)shared, (const T*)h, pass_weight, top, width, scale_output);
    });
    return ti_check_launch("expert_combine");
}
