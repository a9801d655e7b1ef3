// A mixture of gated feed-forward experts of which every token uses a few.
//
//   router    z = Wr y + br (fp32 sums whatever the storage type); the `top` largest z (the lowest index among
//             equals); weights = softmax over those alone
//   expert e  a_e = silu(Wg_e y) * (Wu_e y);  o_e = Wd_e a_e
//   result    h (+)= sum over the chosen experts, in the order in which they were chosen, of weight_e o_e
//
// The experts' matrices lie stacked: gate and up as [experts, ff, width] each, down as [experts, width, ff].
//
// Two ways through the experts.  Token-major (steps of few tokens, and the 32-bit path): a block per (token, chosen
// expert) and slab of the expert's rows; the token's row stands in shared memory as fp32 and every warp forms whole
// dot products with 16-byte loads of the weights, so a weight is read once per token that uses it and nothing is
// gathered or scattered.  Expert-major (long steps, bf16): the (token, expert) pairs are sorted by expert, every
// expert's rows filled up to whole tiles of 128, the tokens' rows gathered in that order, and two tensor-core products
// run over the tiles, each tile against its own expert's weights (ferris_gemm_grouped_tcgen05); a last pass adds every
// token's results, in the order of its choices, into the residual rows.  The kernels here sort, gather and add.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int MOE_MAX_EXPERTS = 1024;
constexpr int MOE_MAX_TOP = 32;

// dot product of a weight row with a row held in shared memory as fp32; 16-byte loads where `vec`; every lane gets the sum
__device__ __forceinline__ float dot_row(const float* __restrict__ w, const float* xs, int n, int lane, bool vec) {
    float acc = 0.0f;
    if (vec) {
        const float4* w4 = reinterpret_cast<const float4*>(w);
        for (int i = lane; i < (n >> 2); i += 32) {
            const float4 a = w4[i];
            const float4 x = *reinterpret_cast<const float4*>(xs + 4 * i);
            acc = fmaf(a.x, x.x, fmaf(a.y, x.y, fmaf(a.z, x.z, fmaf(a.w, x.w, acc))));
        }
    } else {
        for (int i = lane; i < n; i += 32) acc = fmaf(w[i], xs[i], acc);
    }
    return warp_sum(acc);
}
__device__ __forceinline__ float dot_row(const bf16* __restrict__ w, const float* xs, int n, int lane, bool vec) {
    float acc = 0.0f;
    if (vec) {
        const uint4* w8 = reinterpret_cast<const uint4*>(w);
        for (int i = lane; i < (n >> 3); i += 32) {
            const uint4 a = w8[i];
            const float4 x0 = *reinterpret_cast<const float4*>(xs + 8 * i);
            const float4 x1 = *reinterpret_cast<const float4*>(xs + 8 * i + 4);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&a);
            const float2 f0 = __bfloat1622float2(p[0]), f1 = __bfloat1622float2(p[1]);
            const float2 f2 = __bfloat1622float2(p[2]), f3 = __bfloat1622float2(p[3]);
            acc = fmaf(f0.x, x0.x, fmaf(f0.y, x0.y, fmaf(f1.x, x0.z, fmaf(f1.y, x0.w, acc))));
            acc = fmaf(f2.x, x1.x, fmaf(f2.y, x1.y, fmaf(f3.x, x1.z, fmaf(f3.y, x1.w, acc))));
        }
    } else {
        for (int i = lane; i < n; i += 32) acc = fmaf(to_float(w[i]), xs[i], acc);
    }
    return warp_sum(acc);
}
template <typename T>
__device__ __forceinline__ bool rows_vectorise(const T* w, int n) {
    return n % (16 / (int)sizeof(T)) == 0 && ((uintptr_t)w & 15) == 0;
}

// ------------------------------------------------------------------------------------------ router
// A warp per token: logits of all experts (fp32), then `top` rounds of "the largest that is left".
template <typename T>
__global__ void __launch_bounds__(128) moe_router_kernel(const T* x, int ldx, const T* __restrict__ w,
                                                         const float* __restrict__ bias, int* __restrict__ ids,
                                                         float* __restrict__ weights, int tokens, int width, int experts,
                                                         int top) {
    extern __shared__ __align__(16) float smem[];  // per warp: the token's row (width) and its logits (experts)
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * 4 + warp;
    if (t >= tokens) return;
    float* xs = smem + (size_t)warp * (width + experts);
    float* z = xs + width;
    const T* xr = x + (size_t)t * ldx;
    for (int i = lane; i < width; i += 32) xs[i] = to_float(xr[i]);
    __syncwarp();
    const bool vec = rows_vectorise(w, width) && ((uintptr_t)xs & 15) == 0;
    for (int e = 0; e < experts; ++e) {
        const float dot = dot_row(w + (size_t)e * width, xs, width, lane, vec);
        if (lane == 0) z[e] = dot + (bias ? bias[e] : 0.0f);
    }
    __syncwarp();
    float chosen_z = 0.0f, first_z = 0.0f, sum = 0.0f;  // lane s keeps the s-th choice
    int chosen = 0;
    for (int s = 0; s < top; ++s) {
        float best = -INFINITY;
        int at = experts;
        for (int e = lane; e < experts; e += 32) {
            const float v = z[e];
            if (v > best) best = v, at = e;  // ascending e: the lowest index among a lane's equals
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) best = ob, at = oa;
        }
        if (at >= experts) at = s < experts ? s : 0, best = 0.0f;  // only where logits are not numbers
        if (s == 0) first_z = best;
        if (lane == (s & 31) && s < 32) chosen = at, chosen_z = best;
        sum += expf(best - first_z);  // the first choice is the largest: the softmax's maximum
        if (lane == 0) z[at] = -INFINITY;
        __syncwarp();
    }
    if (lane < top) {
        ids[(size_t)t * top + lane] = chosen;
        weights[(size_t)t * top + lane] = expf(chosen_z - first_z) / sum;
    }
}

// ------------------------------------------------------------------------------------------ token-major experts
// act[(t, s), j] = silu(Wg_e[j] . y_t) * (Wu_e[j] . y_t) for e = ids[t, s]; a block per (t, s) and slab of `slab` rows j.
template <typename T>
__global__ void __launch_bounds__(128) moe_gate_up_kernel(const T* x, int ldx, const T* __restrict__ gate,
                                                          const T* __restrict__ up, size_t expert_stride, const int* ids,
                                                          T* __restrict__ act, int width, int ff, int top, int slab) {
    extern __shared__ __align__(16) float xs[];  // the token's row
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pair = blockIdx.x, t = pair / top, e = ids[pair];
    const T* xr = x + (size_t)t * ldx;
    for (int i = threadIdx.x; i < width; i += blockDim.x) xs[i] = to_float(xr[i]);
    __syncthreads();
    const T* g = gate + (size_t)e * expert_stride;
    const T* u = up + (size_t)e * expert_stride;
    const bool vec = rows_vectorise(g, width) && rows_vectorise(u, width);
    const int j0 = blockIdx.y * slab, j1 = min(ff, j0 + slab);
    for (int j = j0 + warp; j < j1; j += 4) {
        const float a = dot_row(g + (size_t)j * width, xs, width, lane, vec);
        const float b = dot_row(u + (size_t)j * width, xs, width, lane, vec);
        if (lane == 0) act[(size_t)pair * ff + j] = from_float<T>((a / (1.0f + expf(-a))) * b);
    }
}

// h[t, c] (+)= sum_s weights[t, s] * (Wd_e(s)[c] . act[(t, s)]); a block per token and slab of `slab` columns c.
template <typename T>
__global__ void __launch_bounds__(128) moe_down_kernel(const T* act, const T* __restrict__ down, const int* ids,
                                                       const float* weights, float* h, int ldh, int width, int ff, int top,
                                                       int slab, int accumulate) {
    extern __shared__ __align__(16) float as[];  // the token's activations: top x ff
    __shared__ int es[MOE_MAX_TOP];
    __shared__ float ws[MOE_MAX_TOP];
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x;
    const T* ar = act + (size_t)t * top * ff;
    for (int i = threadIdx.x; i < top * ff; i += blockDim.x) as[i] = to_float(ar[i]);
    if (threadIdx.x < top) es[threadIdx.x] = ids[(size_t)t * top + threadIdx.x], ws[threadIdx.x] = weights[(size_t)t * top + threadIdx.x];
    __syncthreads();
    const bool vec = rows_vectorise(down, ff) && (ff * sizeof(float)) % 16 == 0;
    const int c0 = blockIdx.y * slab, c1 = min(width, c0 + slab);
    for (int c = c0 + warp; c < c1; c += 4) {
        float sum = 0.0f;
        for (int s = 0; s < top; ++s) {
            const T* row = down + ((size_t)es[s] * width + c) * ff;
            sum = fmaf(ws[s], dot_row(row, as + (size_t)s * ff, ff, lane, vec), sum);
        }
        if (lane == 0) {
            float* dst = h + (size_t)t * ldh + c;
            *dst = accumulate ? *dst + sum : sum;
        }
    }
}

// ------------------------------------------------------------------------------------------ expert-major: sort
// One block.  pos[pair] = the row of pair (t, s) in the sorted order; row_token[row] = its token, or -1 for a row that
// only fills a tile up; tile_expert[tile] = the expert of the tile's rows, or -1 beyond the last row.
constexpr int MOE_TILE = 128;
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* ids, int* pos, int* row_token, int* tile_expert,
                                                        int pairs, int top, int experts, int max_rows) {
    __shared__ int count[MOE_MAX_EXPERTS];
    __shared__ int first[MOE_MAX_EXPERTS + 1];
    pdl_wait();
    pdl_launch_dependents();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    for (int r = threadIdx.x; r < max_rows; r += blockDim.x) row_token[r] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) pos[i] = atomicAdd(&count[ids[i]], 1);  // its rank, for now
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < experts; ++e) {
            first[e] = at;
            at += (count[e] + MOE_TILE - 1) / MOE_TILE * MOE_TILE;
        }
        first[experts] = at;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int row = first[ids[i]] + pos[i];
        pos[i] = row;
        row_token[row] = i / top;
    }
    for (int tile = threadIdx.x; tile < max_rows / MOE_TILE; tile += blockDim.x) {
        const int row = tile * MOE_TILE;
        int e = -1;
        if (row < first[experts]) {
            int lo = 0, hi = experts - 1;  // the last expert whose first row is at or before this tile's
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (first[mid] <= row) lo = mid; else hi = mid - 1;
            }
            e = lo;
        }
        tile_expert[tile] = e;
    }
}

// xs[row] = x[row_token[row]], 16 bytes a thread; rows that fill a tile up are zeroed.
__global__ void __launch_bounds__(256) moe_gather_kernel(const uint4* x, int ldx16, const int* row_token, uint4* xs,
                                                         int rows, int width16) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t n = (size_t)rows * width16;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const int row = (int)(e / width16), i = (int)(e % width16);
        const int t = row_token[row];
        xs[e] = t >= 0 ? x[(size_t)t * ldx16 + i] : make_uint4(0u, 0u, 0u, 0u);
    }
}

// h[t] (+)= sum_s weights[t, s] * y[pos[t, s]], in the order of the choices; four columns a thread.
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* y, int ldy, const int* pos, const float* weights,
                                                          float* h, int ldh, int tokens, int width4, int top,
                                                          int accumulate) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t n = (size_t)tokens * width4;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(e / width4), i = (int)(e % width4);
        float4* dst = reinterpret_cast<float4*>(h + (size_t)t * ldh) + i;
        float4 acc = accumulate ? *dst : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int s = 0; s < top; ++s) {
            const float w = weights[(size_t)t * top + s];
            const float4 v = reinterpret_cast<const float4*>(y + (size_t)pos[(size_t)t * top + s] * ldy)[i];
            sum.x = fmaf(w, v.x, sum.x), sum.y = fmaf(w, v.y, sum.y), sum.z = fmaf(w, v.z, sum.z), sum.w = fmaf(w, v.w, sum.w);
        }
        acc.x += sum.x, acc.y += sum.y, acc.z += sum.z, acc.w += sum.w;
        *dst = acc;
    }
}

}  // namespace

extern "C" int ferris_gemm_grouped_tcgen05(const void* x, const void* w, void* out, int mode, int rows, int N, int K,
                                           int ldx, int ldw, int ldo, int experts, int expert_rows, int up_row_offset,
                                           const int* tile_expert, void* stream);

// Rows of the sorted order that `tokens` tokens choosing `top` of `experts` can need at most (whole tiles of 128).
FERRIS_API int ferris_moe_sorted_rows(int tokens, int top, int experts) {
    const long long pairs = (long long)tokens * top;
    const long long rows = (pairs + MOE_TILE - 1) / MOE_TILE * MOE_TILE + (long long)(experts < pairs ? experts : pairs) * MOE_TILE;
    return rows > 2147483647LL ? -1 : (int)rows;
}

// The experts of a long step in bf16.  x bf16 [tokens, width] rows ldx apart; gate_up bf16 [experts, 2 ff, width] (an
// expert's gate rows, then its up rows); down bf16 [experts, width, ff]; ids, weights [tokens, top]; h fp32.
// Scratch, all sized for rows = ferris_moe_sorted_rows(...): pos int32 [tokens x top], row_token int32 [rows],
// tile_expert int32 [rows / 128], xs bf16 [rows, width], act bf16 [rows, ff], y fp32 [rows, width].
FERRIS_API int ferris_moe_experts_grouped(const void* x, int ldx, const void* gate_up, const void* down, const int* ids,
                                          const float* weights, float* h, int ldh, int tokens, int width, int ff, int top,
                                          int experts, int rows, int* pos, int* row_token, int* tile_expert, void* xs,
                                          void* act, float* y, int accumulate, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (experts <= 0 || experts > MOE_MAX_EXPERTS || top <= 0 || top > experts)
        FERRIS_REFUSE("experts: %d of %d experts", top, experts);
    if (rows != ferris_moe_sorted_rows(tokens, top, experts)) FERRIS_REFUSE("experts: scratch for %d rows", rows);
    if (width % 8 || ff % 8 || ldx % 8 || ldh % 4 || (((uintptr_t)x | (uintptr_t)xs | (uintptr_t)y | (uintptr_t)h) & 15))
        FERRIS_REFUSE("experts: width %d, ff %d and the rows must be multiples of 8 elements and start on 16 bytes", width, ff);
    cudaStream_t s = (cudaStream_t)stream;
    ferris_launch(moe_sort_kernel, dim3(1), dim3(1024), 0, s, ids, pos, row_token, tile_expert, tokens * top, top, experts,
                  rows);
    const size_t n16 = (size_t)rows * (width / 8);
    const size_t want = (n16 + 255) / 256;
    ferris_launch(moe_gather_kernel, dim3((unsigned)(want < 148 * 16 ? want : 148 * 16)), dim3(256), 0, s, (const uint4*)x,
                  ldx / 8, (const int*)row_token, (uint4*)xs, rows, width / 8);
    int rc = ferris_gemm_grouped_tcgen05(xs, gate_up, act, 3, rows, ff, width, width, width, ff, experts, 2 * ff, ff,
                                         tile_expert, stream);
    if (rc != FERRIS_OK) return rc;
    rc = ferris_gemm_grouped_tcgen05(act, down, y, 1, rows, width, ff, ff, ff, width, experts, width, 0, tile_expert, stream);
    if (rc != FERRIS_OK) return rc;
    const size_t n4 = (size_t)tokens * (width / 4);
    const size_t want4 = (n4 + 255) / 256;
    ferris_launch(moe_combine_kernel, dim3((unsigned)(want4 < 148 * 16 ? want4 : 148 * 16)), dim3(256), 0, s, (const float*)y,
                  width, (const int*)pos, weights, h, ldh, tokens, width / 4, top, accumulate);
    FERRIS_LAUNCH_CHECK();
}

FERRIS_API int ferris_moe_router(const void* x, int ldx, int dtype, const void* w, const float* bias, int* ids,
                                 float* weights, int tokens, int width, int experts, int top, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (experts <= 0 || experts > MOE_MAX_EXPERTS || top <= 0 || top > experts || top > MOE_MAX_TOP || width <= 0)
        FERRIS_REFUSE("router: %d experts (at most %d), %d chosen (at most %d), width %d", experts, MOE_MAX_EXPERTS, top,
                      MOE_MAX_TOP, width);
    const size_t smem = 4 * (size_t)(width + experts) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((tokens + 3) / 4), block(128);
    int rc;
    if (dtype == FERRIS_F32) {
        if ((rc = ferris_allow_dynamic_smem((const void*)moe_router_kernel<float>, smem)) != FERRIS_OK) return rc;
        ferris_launch(moe_router_kernel<float>, grid, block, smem, s, (const float*)x, ldx, (const float*)w, bias, ids,
                      weights, tokens, width, experts, top);
    } else if (dtype == FERRIS_BF16) {
        if ((rc = ferris_allow_dynamic_smem((const void*)moe_router_kernel<bf16>, smem)) != FERRIS_OK) return rc;
        ferris_launch(moe_router_kernel<bf16>, grid, block, smem, s, (const bf16*)x, ldx, (const bf16*)w, bias, ids, weights,
                      tokens, width, experts, top);
    } else
        FERRIS_REFUSE("router: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}

// x [tokens, width] rows ldx apart; gate, up: expert e's [ff, width] matrices lie gate_up_stride elements after expert
// e - 1's (two tensors, or the two halves of one [experts, 2 ff, width]); down [experts, width, ff]; ids int32 and
// weights fp32 [tokens, top]; act [tokens x top, ff] (scratch, the activations' type); h fp32 rows ldh apart.
FERRIS_API int ferris_moe_experts_token_major(const void* x, int ldx, int dtype, const void* gate, const void* up,
                                              long long gate_up_stride, const void* down, const int* ids,
                                              const float* weights, void* act, float* h,
                                              int ldh, int tokens, int width, int ff, int top, int accumulate,
                                              void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (width <= 0 || ff <= 0 || top <= 0 || top > MOE_MAX_TOP) FERRIS_REFUSE("experts: width %d, ff %d, %d chosen", width, ff, top);
    const size_t smem_up = (size_t)width * sizeof(float), smem_down = (size_t)top * ff * sizeof(float);
    if (smem_up > 200 * 1024 || smem_down > 200 * 1024)
        FERRIS_REFUSE("experts: a row of %d or %d x %d activations do not fit shared memory", width, top, ff);
    if ((long long)tokens * top > 2147483647LL / 2) FERRIS_REFUSE("experts: %d tokens are more than one launch takes", tokens);
    cudaStream_t s = (cudaStream_t)stream;
    // slabs of rows: enough blocks to fill the SMs a few times over, at least 4 rows (a row per warp) each
    const int pairs = tokens * top;
    auto slab_of = [](int rows, int blocks_other) {
        int slab = 32;
        while (slab > 4 && (long long)blocks_other * ((rows + slab - 1) / slab) < 148 * 4) slab >>= 1;
        return slab;
    };
    const int slab_up = slab_of(ff, pairs), slab_down = slab_of(width, tokens);
    const dim3 grid_up(pairs, (ff + slab_up - 1) / slab_up), grid_down(tokens, (width + slab_down - 1) / slab_down);
    if (grid_up.y > 65535 || grid_down.y > 65535) FERRIS_REFUSE("experts: too many slabs");
    int rc;
#define FERRIS_MOE_RUN(T)                                                                                                 \
    do {                                                                                                                  \
        if ((rc = ferris_allow_dynamic_smem((const void*)moe_gate_up_kernel<T>, smem_up)) != FERRIS_OK) return rc;        \
        if ((rc = ferris_allow_dynamic_smem((const void*)moe_down_kernel<T>, smem_down)) != FERRIS_OK) return rc;         \
        ferris_launch(moe_gate_up_kernel<T>, dim3(grid_up.x, grid_up.y, 1), dim3(128), smem_up, s, (const T*)x, ldx,      \
                      (const T*)gate, (const T*)up, (size_t)gate_up_stride, ids, (T*)act, width, ff, top, slab_up);                                    \
        ferris_launch(moe_down_kernel<T>, grid_down, dim3(128), smem_down, s, (const T*)act, (const T*)down, ids, weights, \
                      h, ldh, width, ff, top, slab_down, accumulate);                                                     \
    } while (0)
    if (dtype == FERRIS_F32)
        FERRIS_MOE_RUN(float);
    else if (dtype == FERRIS_BF16)
        FERRIS_MOE_RUN(bf16);
    else
        FERRIS_REFUSE("experts: unknown dtype %d", dtype);
#undef FERRIS_MOE_RUN
    FERRIS_LAUNCH_CHECK();
}
