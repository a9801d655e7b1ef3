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
// gathered or scattered.  Expert-major (long steps, bf16): see moe_grouped.cu.
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
                                                          const T* __restrict__ up, const int* ids, T* __restrict__ act,
                                                          int width, int ff, int top, int slab) {
    extern __shared__ __align__(16) float xs[];  // the token's row
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pair = blockIdx.x, t = pair / top, e = ids[pair];
    const T* xr = x + (size_t)t * ldx;
    for (int i = threadIdx.x; i < width; i += blockDim.x) xs[i] = to_float(xr[i]);
    __syncthreads();
    const T* g = gate + (size_t)e * ff * width;
    const T* u = up + (size_t)e * ff * width;
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

}  // namespace

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

// x [tokens, width] rows ldx apart; gate, up [experts, ff, width]; down [experts, width, ff]; ids int32 and weights
// fp32 [tokens, top]; act [tokens x top, ff] (scratch, the activations' type); h fp32 rows ldh apart.
FERRIS_API int ferris_moe_experts_token_major(const void* x, int ldx, int dtype, const void* gate, const void* up,
                                              const void* down, const int* ids, const float* weights, void* act, float* h,
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
                      (const T*)gate, (const T*)up, ids, (T*)act, width, ff, top, slab_up);                                    \
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
