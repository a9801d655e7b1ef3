// A mixture of gated feed-forward experts of which every token uses a few.
//
//   router    z = Wr y + br (fp32 sums whatever the storage type); the `top` largest z (the lowest index among
//             equals); weights = softmax over those alone
//   expert e  a_e = silu(Wg_e y) * (Wu_e y);  o_e = Wd_e a_e
//   result    h (+)= sum over the chosen experts, in the order in which they were chosen, of weight_e o_e
//
// A second kind of router (`scored`): s = softmax(z) over ALL router outputs; the choice is made by c = s + correction
// (a learned number per output), the outputs stand in `groups` equal groups of neighbours of which only the `keep`
// with the largest c in them take part (the others count as minus infinity), the `top` largest c are chosen (the
// lowest index among equals) and their weights are s / (sum of the chosen s + 1e-20).  Router outputs beyond the
// experts with weights are identity experts, whose result is the token's row itself: the router hands them on as one
// index past the last expert, which every expert kernel skips, and leaves the sum of their weights per token, which
// the adding passes multiply the token's row by.  The experts' gated activation is one of the kinds of
// ferris_gated_act.
//
// The experts' matrices lie stacked: gate and up as [experts, ff, width] each, down as [experts, width, ff].
//
// Three ways through the experts.  Token-major (a single choice; the 32-bit path of long steps): a block per (token, chosen expert) and
// slab of the expert's rows; the token's row stands in shared memory as fp32 and every warp forms whole dot products
// with 16-byte loads of the weights, so a weight is read once per token that uses it and nothing is gathered or
// scattered.  Expert-major for few tokens (decode steps): a block per (expert, slab of rows) finds the tokens that
// chose its expert, holds four of their rows in shared memory at a time and forms the same dot products for all four
// from one pass over the weight rows, which every lane streams through shared memory with asynchronous 16-byte copies
// a few steps ahead; a last pass adds every token's results in the order of its choices.  Both give a token the same
// bits.  Expert-major (long steps, bf16): the (token, expert) pairs are sorted by expert, every
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
// 16 bytes of a weight row as fp32: four elements of float, eight of bf16
__device__ __forceinline__ void load_chunk(const float* w, int i, float (&f)[4]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(w) + i);
    f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w;
}
__device__ __forceinline__ void load_chunk(const bf16* w, int i, float (&f)[8]) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(w) + i);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float2 v = __bfloat1622float2(p[q]);
        f[2 * q] = v.x, f[2 * q + 1] = v.y;
    }
}
// R weight rows against M rows in shared memory (fp32, `xstride` apart): the R loads of a step are in flight together
// and serve all M rows.  Every sum is formed in the order of dot_row, so a result depends on neither R nor M.
template <int R, int M, typename T>
__device__ __forceinline__ void dot_tile(const T* const (&w)[R], const float* xs, int xstride, int n, int lane, bool vec,
                                         float (&out)[R][M]) {
    constexpr int C = 16 / (int)sizeof(T);
    float acc[R][M];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) acc[r][m] = 0.0f;
    if (vec) {
        for (int i = lane; i < n / C; i += 32) {
            float f[R][C];
#pragma unroll
            for (int r = 0; r < R; ++r) load_chunk(w[r], i, f[r]);
#pragma unroll
            for (int m = 0; m < M; ++m) {
#pragma unroll
                for (int q = 0; q < C; q += 4) {
                    const float4 x = *reinterpret_cast<const float4*>(xs + (size_t)m * xstride + C * i + q);
#pragma unroll
                    for (int r = 0; r < R; ++r)
                        acc[r][m] = fmaf(f[r][q], x.x, fmaf(f[r][q + 1], x.y, fmaf(f[r][q + 2], x.z, fmaf(f[r][q + 3], x.w, acc[r][m]))));
                }
            }
        }
    } else {
        for (int i = lane; i < n; i += 32) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float a = to_float(w[r][i]);
#pragma unroll
                for (int m = 0; m < M; ++m) acc[r][m] = fmaf(a, xs[(size_t)m * xstride + i], acc[r][m]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) out[r][m] = warp_sum(acc[r][m]);
}
// The same sums with the weights streamed through shared memory: every lane copies its own 16-byte pieces of the R
// rows asynchronously into slots that only it reads back (so nothing but its own copy groups orders them), FEW_STAGES
// steps ahead.  The bytes in flight are then bounded by shared memory, not by registers.  Needs the 16-byte form (vec).
constexpr int FEW_STAGES = 4;
constexpr int FEW_RING_BYTES = FEW_STAGES * 4 * 512;  // per warp: stages x up to 4 rows x 32 lanes x 16 bytes
__device__ __forceinline__ void copy16_async(void* smem_dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void copy_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void chunk_to_float(const uint4& a, float (&f)[4], const float*) {
    f[0] = __uint_as_float(a.x), f[1] = __uint_as_float(a.y), f[2] = __uint_as_float(a.z), f[3] = __uint_as_float(a.w);
}
__device__ __forceinline__ void chunk_to_float(const uint4& a, float (&f)[8], const bf16*) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float2 v = __bfloat1622float2(p[q]);
        f[2 * q] = v.x, f[2 * q + 1] = v.y;
    }
}
template <int R, int M, typename T>
__device__ __forceinline__ void dot_tile_streamed(const T* const (&w)[R], const float* xs, int xstride, int n, int lane,
                                                  uint4* ring, float (&out)[R][M]) {
    constexpr int C = 16 / (int)sizeof(T);
    static_assert(R <= 4, "a warp's slots hold four rows");
    const int chunks = n / C;
    float acc[R][M];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) acc[r][m] = 0.0f;
    uint4* mine = ring + lane;  // slot (stage, r) at mine[(stage * 4 + r) * 32]
#pragma unroll
    for (int st = 0; st < FEW_STAGES; ++st) {
        const int i = lane + 32 * st;
        if (i < chunks) {
#pragma unroll
            for (int r = 0; r < R; ++r) copy16_async(mine + (st * 4 + r) * 32, reinterpret_cast<const uint4*>(w[r]) + i);
        }
        copy_commit();
    }
    int st = 0;
    for (int i = lane; i < chunks; i += 32) {
        copy_wait<FEW_STAGES - 1>();
        float f[R][C];
#pragma unroll
        for (int r = 0; r < R; ++r) chunk_to_float(mine[(st * 4 + r) * 32], f[r], (const T*)nullptr);
#pragma unroll
        for (int m = 0; m < M; ++m) {
#pragma unroll
            for (int q = 0; q < C; q += 4) {
                const float4 x = *reinterpret_cast<const float4*>(xs + (size_t)m * xstride + C * i + q);
#pragma unroll
                for (int r = 0; r < R; ++r)
                    acc[r][m] = fmaf(f[r][q], x.x, fmaf(f[r][q + 1], x.y, fmaf(f[r][q + 2], x.z, fmaf(f[r][q + 3], x.w, acc[r][m]))));
            }
        }
        const int next = i + 32 * FEW_STAGES;  // the slot is read: it takes the piece FEW_STAGES steps on
        if (next < chunks) {
#pragma unroll
            for (int r = 0; r < R; ++r) copy16_async(mine + (st * 4 + r) * 32, reinterpret_cast<const uint4*>(w[r]) + next);
        }
        copy_commit();
        st = st + 1 == FEW_STAGES ? 0 : st + 1;
    }
    copy_wait<0>();
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) out[r][m] = warp_sum(acc[r][m]);
}
// streamed where the rows take 16-byte pieces, else element by element
template <int R, int M, typename T>
__device__ __forceinline__ void dot_tile_few(const T* const (&w)[R], const float* xs, int xstride, int n, int lane, bool vec,
                                             uint4* ring, float (&out)[R][M]) {
    if (vec)
        dot_tile_streamed<R, M>(w, xs, xstride, n, lane, ring, out);
    else
        dot_tile<R, M>(w, xs, xstride, n, lane, false, out);
}
template <int R, typename T>
__device__ __forceinline__ void dot_rows(const T* const (&w)[R], const float* xs, int n, int lane, bool vec, float (&out)[R]) {
    float d[R][1];
    dot_tile<R, 1>(w, xs, 0, n, lane, vec, d);
#pragma unroll
    for (int r = 0; r < R; ++r) out[r] = d[r][0];
}
template <typename T>
__device__ __forceinline__ bool rows_vectorise(const T* w, int n) {
    return n % (16 / (int)sizeof(T)) == 0 && ((uintptr_t)w & 15) == 0;
}

// dst[0..n) (shared memory, fp32, 16-byte aligned) = src[0..n), by threads `me` of `threads`; 16-byte loads, several in
// flight, where the row allows them.  The source is not written while the kernel runs.
template <typename T>
__device__ __forceinline__ void stage_row(float* dst, const T* src, int n, int me, int threads) {
    constexpr int C = 16 / (int)sizeof(T);
    if (n % C == 0 && ((uintptr_t)src & 15) == 0) {
#pragma unroll 4
        for (int i = me; i < n / C; i += threads) {
            float f[C];
            load_chunk(src, i, f);
#pragma unroll
            for (int q = 0; q < C; q += 4)
                *reinterpret_cast<float4*>(dst + C * i + q) = make_float4(f[q], f[q + 1], f[q + 2], f[q + 3]);
        }
    } else {
#pragma unroll 4
        for (int i = me; i < n; i += threads) dst[i] = to_float(src[i]);
    }
}

// ------------------------------------------------------------------------------------------ router
// Logits of all experts (fp32), then `top` rounds of "the largest that is left".  A warp per token; in steps of few
// tokens (BLOCK) a block per token, whose four warps share the experts' dot products (each formed by one warp in the
// same order either way, so a token's logits do not depend on the form) and whose first warp then chooses.
template <typename T, bool BLOCK>
__global__ void __launch_bounds__(128) moe_router_kernel(const T* x, int ldx, const T* __restrict__ w,
                                                         const float* __restrict__ bias, int* __restrict__ ids,
                                                         float* __restrict__ weights, int tokens, int width, int experts,
                                                         int top, int scored, const float* __restrict__ correction,
                                                         int groups, int keep, int with_weights,
                                                         float* __restrict__ identity_w) {
    extern __shared__ __align__(16) float smem[];  // per warp (per block): the token's row (width), its logits (experts), and for the scored kind the choice scores (experts) and the groups' (experts at most)
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = BLOCK ? blockIdx.x : blockIdx.x * 4 + warp;
    if (t >= tokens) return;
    float* xs = smem + (BLOCK ? 0 : (size_t)warp * ((width + 3 * experts + 3) & ~3));  // every warp's row starts on 16 bytes
    float* z = xs + width;
    const T* xr = x + (size_t)t * ldx;
    if (BLOCK) {
        stage_row(xs, xr, width, threadIdx.x, blockDim.x);
        __syncthreads();
    } else {
        stage_row(xs, xr, width, lane, 32);
        __syncwarp();
    }
    const bool vec = rows_vectorise(w, width) && ((uintptr_t)xs & 15) == 0;
    for (int e = BLOCK ? warp : 0; e < experts; e += BLOCK ? 4 : 1) {
        const float dot = dot_row(w + (size_t)e * width, xs, width, lane, vec);
        if (lane == 0) z[e] = dot + (bias ? bias[e] : 0.0f);
    }
    if (BLOCK) {
        __syncthreads();
        if (warp) return;
    } else {
        __syncwarp();
    }
    if (scored) {
        float* c = z + experts;
        float* gsc = c + experts;
        float mx = -INFINITY;
        for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, z[e]);
        mx = warp_max(mx);
        float total = 0.0f;
        for (int e = lane; e < experts; e += 32) total += expf(z[e] - mx);
        total = warp_sum(total);
        for (int e = lane; e < experts; e += 32) {
            const float p = expf(z[e] - mx) / total;
            z[e] = p, c[e] = p + (correction ? correction[e] : 0.0f);
        }
        __syncwarp();
        const int size = experts / groups;
        if (keep < groups) {
            for (int g = lane; g < groups; g += 32) {
                float best = -INFINITY;
                for (int j = 0; j < size; ++j) best = fmaxf(best, c[g * size + j]);
                gsc[g] = best;
            }
            __syncwarp();
            for (int round = 0; round < keep; ++round) {  // the best group that is left; +inf marks a group that stays
                float best = -INFINITY;
                int at = groups;
                for (int g = lane; g < groups; g += 32) {
                    const float v = gsc[g];
                    if (v != INFINITY && (v > best || at == groups)) best = v, at = g;
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                    const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                    if (oa < groups && (at == groups || ob > best || (ob == best && oa < at))) best = ob, at = oa;
                }
                if (lane == 0 && at < groups) gsc[at] = INFINITY;
                __syncwarp();
            }
            for (int e = lane; e < experts; e += 32)
                if (gsc[e / size] != INFINITY) c[e] = -INFINITY;
            __syncwarp();
        }
        float chosen_p = 0.0f;
        int chosen = 0;
        for (int s = 0; s < top; ++s) {
            float best = -INFINITY;
            int at = experts;
            for (int e = lane; e < experts; e += 32) {
                const float v = c[e];
                if (v > best) best = v, at = e;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa < at)) best = ob, at = oa;
            }
            if (at >= experts) at = s < experts ? s : 0;  // only where scores are not numbers
            if (lane == (s & 31) && s < 32) chosen = at, chosen_p = z[at];
            if (lane == 0) c[at] = -INFINITY;
            __syncwarp();
        }
        const float denom = warp_sum(lane < top ? chosen_p : 0.0f) + 1e-20f;
        const float wgt = chosen_p / denom;
        const bool identity = lane < top && chosen >= with_weights;
        const float idw = warp_sum(identity ? wgt : 0.0f);
        if (lane < top) {
            ids[(size_t)t * top + lane] = identity ? with_weights : chosen;
            weights[(size_t)t * top + lane] = wgt;
        }
        if (identity_w && lane == 0) identity_w[t] = idw;
        return;
    }
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
                                                          T* __restrict__ act, int width, int ff, int top, int slab,
                                                          int experts, int act_kind, float act_limit) {
    extern __shared__ __align__(16) float xs[];  // the token's row
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pair = blockIdx.x, t = pair / top, e = ids[pair];
    if (e >= experts) return;  // an identity expert: nothing to form
    const T* xr = x + (size_t)t * ldx;
    stage_row(xs, xr, width, threadIdx.x, blockDim.x);
    __syncthreads();
    const T* g = gate + (size_t)e * expert_stride;
    const T* u = up + (size_t)e * expert_stride;
    const bool vec = rows_vectorise(g, width) && rows_vectorise(u, width);
    const int j0 = blockIdx.y * slab, j1 = min(ff, j0 + slab);
    // a warp takes rows j and j + 4 of both matrices at a time: four weight rows in flight for one read of the token's row
    for (int j = j0 + warp; j < j1; j += 8) {
        if (j + 4 < j1) {
            const T* const rows[4] = {g + (size_t)j * width, u + (size_t)j * width, g + (size_t)(j + 4) * width,
                                      u + (size_t)(j + 4) * width};
            float d[4];
            dot_rows<4>(rows, xs, width, lane, vec, d);
            if (lane == 0) {
                act[(size_t)pair * ff + j] = from_float<T>(ferris_gated_act(d[0], d[1], act_kind, act_limit));
                act[(size_t)pair * ff + j + 4] = from_float<T>(ferris_gated_act(d[2], d[3], act_kind, act_limit));
            }
        } else {
            const T* const rows[2] = {g + (size_t)j * width, u + (size_t)j * width};
            float d[2];
            dot_rows<2>(rows, xs, width, lane, vec, d);
            if (lane == 0) act[(size_t)pair * ff + j] = from_float<T>(ferris_gated_act(d[0], d[1], act_kind, act_limit));
        }
    }
}

// h[t, c] (+)= sum_s weights[t, s] * (Wd_e(s)[c] . act[(t, s)]); a block per token and slab of `slab` columns c.
template <typename T>
__global__ void __launch_bounds__(128) moe_down_kernel(const T* act, const T* __restrict__ down, const int* ids,
                                                       const float* weights, float* h, int ldh, int width, int ff, int top,
                                                       int slab, int accumulate, int experts, const T* x, int ldx,
                                                       const float* identity_w) {
    extern __shared__ __align__(16) float as[];  // the token's activations: top x ff
    __shared__ int es[MOE_MAX_TOP];
    __shared__ float ws[MOE_MAX_TOP];
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x;
    const T* ar = act + (size_t)t * top * ff;
    if (threadIdx.x < top) es[threadIdx.x] = ids[(size_t)t * top + threadIdx.x], ws[threadIdx.x] = weights[(size_t)t * top + threadIdx.x];
    __syncthreads();
    for (int s = 0; s < top; ++s)  // the rows of identity experts were never written
        if (es[s] < experts) stage_row(as + (size_t)s * ff, ar + (size_t)s * ff, ff, threadIdx.x, blockDim.x);
    __syncthreads();
    const float idw = identity_w ? identity_w[t] : 0.0f;
    const bool vec = rows_vectorise(down, ff) && (ff * sizeof(float)) % 16 == 0;
    const int c0 = blockIdx.y * slab, c1 = min(width, c0 + slab);
    // a warp takes columns c, c + 4, c + 8 and c + 12 at a time: four weight rows in flight for one read of the activations
    for (int c = c0 + warp; c < c1; c += 16) {
        float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const int n = min(4, (c1 - c + 3) / 4);
        for (int s = 0; s < top; ++s) {
            if (es[s] >= experts) continue;
            const T* first = down + ((size_t)es[s] * width + c) * ff;
            const float* a = as + (size_t)s * ff;
            if (n == 4) {
                const T* const rows[4] = {first, first + (size_t)4 * ff, first + (size_t)8 * ff, first + (size_t)12 * ff};
                float d[4];
                dot_rows<4>(rows, a, ff, lane, vec, d);
#pragma unroll
                for (int r = 0; r < 4; ++r) sum[r] = fmaf(ws[s], d[r], sum[r]);
            } else {
                for (int r = 0; r < n; ++r) sum[r] = fmaf(ws[s], dot_row(first + (size_t)4 * r * ff, a, ff, lane, vec), sum[r]);
            }
        }
        if (lane == 0) {
            for (int r = 0; r < n; ++r) {
                float* dst = h + (size_t)t * ldh + c + 4 * r;
                if (identity_w) sum[r] = fmaf(idw, to_float(x[(size_t)t * ldx + c + 4 * r]), sum[r]);
                *dst = accumulate ? *dst + sum[r] : sum[r];
            }
        }
    }
}

// ------------------------------------------------------------------------------------------ expert-major, few tokens
// Steps of few tokens with the weights read once per expert instead of once per (token, expert): a block per (expert,
// slab of rows) lists the pairs that chose its expert (in the order of the pairs), takes their tokens' rows into shared
// memory four at a time and forms every weight row's dot products with all four from one load of the row.  Blocks of
// experts that nobody chose return at once.  Every sum is formed as in the token-major kernels, bit for bit.
constexpr int MOE_FEW_ROWS = 4;       // token rows in shared memory at a time: a warp stages a row
constexpr int MOE_FEW_MAX_PAIRS = 1024;
constexpr int FEW_WARPS = 8;          // warps a block: they share the token rows

// list[0..n) = the pairs whose expert is e, ascending; returns n (to every thread)
__device__ __forceinline__ int pairs_of_expert(const int* ids, int pairs, int e, int* list, int* count) {
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        int n = 0;
        for (int base = 0; base < pairs; base += 32) {
            const int p = base + lane;
            const bool mine = p < pairs && ids[p] == e;
            const unsigned m = __ballot_sync(0xffffffffu, mine);
            if (mine) list[n + __popc(m & ((1u << lane) - 1u))] = p;
            n += __popc(m);
        }
        if (lane == 0) *count = n;
    }
    __syncthreads();
    return *count;
}

template <typename T, int M>
__device__ __forceinline__ void gate_up_rows(const T* g, const T* u, const float* xs, int width, int ff, int j0, int j1,
                                             const int* pair, T* __restrict__ act, int lane, int warp, bool vec,
                                             uint4* ring, int act_kind, float act_limit) {
    for (int j = j0 + warp; j < j1; j += 2 * FEW_WARPS) {
        if (j + FEW_WARPS < j1) {
            const T* const rows[4] = {g + (size_t)j * width, u + (size_t)j * width, g + (size_t)(j + FEW_WARPS) * width,
                                      u + (size_t)(j + FEW_WARPS) * width};
            float d[4][M];
            dot_tile_few<4, M>(rows, xs, width, width, lane, vec, ring, d);
            if (lane == 0) {
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    act[(size_t)pair[m] * ff + j] = from_float<T>(ferris_gated_act(d[0][m], d[1][m], act_kind, act_limit));
                    act[(size_t)pair[m] * ff + j + FEW_WARPS] = from_float<T>(ferris_gated_act(d[2][m], d[3][m], act_kind, act_limit));
                }
            }
        } else {
            const T* const rows[2] = {g + (size_t)j * width, u + (size_t)j * width};
            float d[2][M];
            dot_tile_few<2, M>(rows, xs, width, width, lane, vec, ring, d);
            if (lane == 0) {
#pragma unroll
                for (int m = 0; m < M; ++m)
                    act[(size_t)pair[m] * ff + j] = from_float<T>(ferris_gated_act(d[0][m], d[1][m], act_kind, act_limit));
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(32 * FEW_WARPS) moe_gate_up_few_kernel(const T* x, int ldx, const T* __restrict__ gate,
                                                              const T* __restrict__ up, size_t expert_stride, const int* ids,
                                                              T* __restrict__ act, int width, int ff, int pairs, int top,
                                                              int slab, int act_kind, float act_limit) {
    extern __shared__ __align__(16) float dyn[];  // every warp's slots for weights in flight, then MOE_FEW_ROWS token rows
    __shared__ int list[MOE_FEW_MAX_PAIRS];
    __shared__ int count;
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint4* ring = reinterpret_cast<uint4*>(dyn) + warp * (FEW_RING_BYTES / 16);
    float* xs = dyn + FEW_WARPS * (FEW_RING_BYTES / 4);
    const int e = blockIdx.x;
    const int n = pairs_of_expert(ids, pairs, e, list, &count);
    if (n == 0) return;
    const T* g = gate + (size_t)e * expert_stride;
    const T* u = up + (size_t)e * expert_stride;
    const bool vec = rows_vectorise(g, width) && rows_vectorise(u, width);
    const int j0 = blockIdx.y * slab, j1 = min(ff, j0 + slab);
    for (int first = 0; first < n; first += MOE_FEW_ROWS) {
        const int m = min(MOE_FEW_ROWS, n - first);
        if (first) __syncthreads();  // the rows before are done with
        // a warp a row, so that the rows' loads are in flight together
        if (warp < m) stage_row(xs + (size_t)warp * width, x + (size_t)(list[first + warp] / top) * ldx, width, lane, 32);
        __syncthreads();
        const int* pair = list + first;
        switch (m) {
            case 1: gate_up_rows<T, 1>(g, u, xs, width, ff, j0, j1, pair, act, lane, warp, vec, ring, act_kind, act_limit); break;
            case 2: gate_up_rows<T, 2>(g, u, xs, width, ff, j0, j1, pair, act, lane, warp, vec, ring, act_kind, act_limit); break;
            case 3: gate_up_rows<T, 3>(g, u, xs, width, ff, j0, j1, pair, act, lane, warp, vec, ring, act_kind, act_limit); break;
            default: gate_up_rows<T, 4>(g, u, xs, width, ff, j0, j1, pair, act, lane, warp, vec, ring, act_kind, act_limit); break;
        }
    }
}

template <typename T, int M>
__device__ __forceinline__ void down_rows(const T* d, const float* as, int width, int ff, int c0, int c1, const int* pair,
                                          float* __restrict__ y, int lane, int warp, bool vec, uint4* ring) {
    for (int c = c0 + warp; c < c1; c += 4 * FEW_WARPS) {
        const int n = min(4, (c1 - c + FEW_WARPS - 1) / FEW_WARPS);
        float sum[4][M];
        if (n == 4) {
            const T* const rows[4] = {d + (size_t)c * ff, d + (size_t)(c + FEW_WARPS) * ff, d + (size_t)(c + 2 * FEW_WARPS) * ff,
                                      d + (size_t)(c + 3 * FEW_WARPS) * ff};
            dot_tile_few<4, M>(rows, as, ff, ff, lane, vec, ring, sum);
        } else {
            for (int r = 0; r < n; ++r) {
                const T* const row[1] = {d + (size_t)(c + FEW_WARPS * r) * ff};
                float one[1][M];
                dot_tile_few<1, M>(row, as, ff, ff, lane, vec, ring, one);
#pragma unroll
                for (int m = 0; m < M; ++m) sum[r][m] = one[0][m];
            }
        }
        if (lane == 0) {
            for (int r = 0; r < n; ++r)
#pragma unroll
                for (int m = 0; m < M; ++m) y[(size_t)pair[m] * width + c + FEW_WARPS * r] = sum[r][m];
        }
    }
}

// y[pair, c] = Wd_e[c] . act[pair] for the pairs of expert e; a block per (expert, slab of columns)
template <typename T>
__global__ void __launch_bounds__(32 * FEW_WARPS) moe_down_few_kernel(const T* act, const T* __restrict__ down, const int* ids,
                                                           float* __restrict__ y, int width, int ff, int pairs, int slab) {
    extern __shared__ __align__(16) float dyn[];  // every warp's slots for weights in flight, then MOE_FEW_ROWS rows of activations
    __shared__ int list[MOE_FEW_MAX_PAIRS];
    __shared__ int count;
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint4* ring = reinterpret_cast<uint4*>(dyn) + warp * (FEW_RING_BYTES / 16);
    float* as = dyn + FEW_WARPS * (FEW_RING_BYTES / 4);
    const int e = blockIdx.x;
    const int n = pairs_of_expert(ids, pairs, e, list, &count);
    if (n == 0) return;
    const T* d = down + (size_t)e * width * ff;
    const bool vec = rows_vectorise(d, ff) && (ff * sizeof(float)) % 16 == 0;
    const int c0 = blockIdx.y * slab, c1 = min(width, c0 + slab);
    for (int first = 0; first < n; first += MOE_FEW_ROWS) {
        const int m = min(MOE_FEW_ROWS, n - first);
        if (first) __syncthreads();
        if (warp < m) stage_row(as + (size_t)warp * ff, act + (size_t)list[first + warp] * ff, ff, lane, 32);
        __syncthreads();
        const int* pair = list + first;
        switch (m) {
            case 1: down_rows<T, 1>(d, as, width, ff, c0, c1, pair, y, lane, warp, vec, ring); break;
            case 2: down_rows<T, 2>(d, as, width, ff, c0, c1, pair, y, lane, warp, vec, ring); break;
            case 3: down_rows<T, 3>(d, as, width, ff, c0, c1, pair, y, lane, warp, vec, ring); break;
            default: down_rows<T, 4>(d, as, width, ff, c0, c1, pair, y, lane, warp, vec, ring); break;
        }
    }
}

// ------------------------------------------------------------------------------------------ expert-major: sort
// One block.  pos[pair] = the row of pair (t, s) in the sorted order; row_token[row] = its token, or -1 for a row that
// only fills a tile up; tile_expert[tile] = the expert of the tile's rows, or -1 beyond the last row.
constexpr int MOE_TILE = 128;
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* ids, int* pos, int* row_token, int* tile_expert,
                                                        int pairs, int top, int experts, int max_rows, int with_weights) {
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
            e = lo < with_weights ? lo : -1;  // the rows of identity experts meet no weights
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

// h[t] (+)= sum_s weights[t, s] * y[pos[t, s]] (without pos: y[t x top + s]), in the order of the choices; four columns
// a thread.
template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* y, int ldy, const int* pos, const float* weights,
                                                          float* h, int ldh, int tokens, int width4, int top,
                                                          int accumulate, const int* ids, int experts, const T* x, int ldx,
                                                          const float* identity_w) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t n = (size_t)tokens * width4;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(e / width4), i = (int)(e % width4);
        float4* dst = reinterpret_cast<float4*>(h + (size_t)t * ldh) + i;
        float4 acc = accumulate ? *dst : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int s = 0; s < top; ++s) {
            if (ids && ids[(size_t)t * top + s] >= experts) continue;  // an identity expert: its row was never written
            const float w = weights[(size_t)t * top + s];
            const size_t row = pos ? (size_t)pos[(size_t)t * top + s] : (size_t)t * top + s;
            const float4 v = reinterpret_cast<const float4*>(y + row * ldy)[i];
            sum.x = fmaf(w, v.x, sum.x), sum.y = fmaf(w, v.y, sum.y), sum.z = fmaf(w, v.z, sum.z), sum.w = fmaf(w, v.w, sum.w);
        }
        if (identity_w) {
            const float w = identity_w[t];
            const T* xr = x + (size_t)t * ldx + 4 * i;
            sum.x = fmaf(w, to_float(xr[0]), sum.x), sum.y = fmaf(w, to_float(xr[1]), sum.y);
            sum.z = fmaf(w, to_float(xr[2]), sum.z), sum.w = fmaf(w, to_float(xr[3]), sum.w);
        }
        acc.x += sum.x, acc.y += sum.y, acc.z += sum.z, acc.w += sum.w;
        *dst = acc;
    }
}

}  // namespace

extern "C" void ferris_gemm_set_gated_activation(int kind, float limit);
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
// identity_w (may be null): fp32 [tokens]; with it, ids may hold `experts` (an identity expert: the pair meets no weights)
// and h also gets identity_w[t] x[t]; the scratch is then sized for experts + 1.  act_kind, act_limit: the gated
// activation (ferris_gated_act).
FERRIS_API int ferris_moe_experts_grouped(const void* x, int ldx, const void* gate_up, const void* down, const int* ids,
                                          const float* weights, float* h, int ldh, int tokens, int width, int ff, int top,
                                          int experts, int rows, int* pos, int* row_token, int* tile_expert, void* xs,
                                          void* act, float* y, int accumulate, int act_kind, float act_limit,
                                          const float* identity_w, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    const int sorted = experts + (identity_w ? 1 : 0);  // the identity experts' pairs sort behind the last expert's
    if (experts <= 0 || sorted > MOE_MAX_EXPERTS || top <= 0 || top > MOE_MAX_TOP)
        FERRIS_REFUSE("experts: %d of %d experts", top, experts);
    if (rows != ferris_moe_sorted_rows(tokens, top, sorted)) FERRIS_REFUSE("experts: scratch for %d rows", rows);
    if (width % 8 || ff % 8 || ldx % 8 || ldh % 4 || (((uintptr_t)x | (uintptr_t)xs | (uintptr_t)y | (uintptr_t)h) & 15))
        FERRIS_REFUSE("experts: width %d, ff %d and the rows must be multiples of 8 elements and start on 16 bytes", width, ff);
    cudaStream_t s = (cudaStream_t)stream;
    ferris_launch(moe_sort_kernel, dim3(1), dim3(1024), 0, s, ids, pos, row_token, tile_expert, tokens * top, top, sorted,
                  rows, experts);
    const size_t n16 = (size_t)rows * (width / 8);
    const size_t want = (n16 + 255) / 256;
    ferris_launch(moe_gather_kernel, dim3((unsigned)(want < 148 * 16 ? want : 148 * 16)), dim3(256), 0, s, (const uint4*)x,
                  ldx / 8, (const int*)row_token, (uint4*)xs, rows, width / 8);
    ferris_gemm_set_gated_activation(act_kind, act_limit);  // taken by the product launched next
    int rc = ferris_gemm_grouped_tcgen05(xs, gate_up, act, 3, rows, ff, width, width, width, ff, experts, 2 * ff, ff,
                                         tile_expert, stream);
    ferris_gemm_set_gated_activation(0, 0.0f);
    if (rc != FERRIS_OK) return rc;
    rc = ferris_gemm_grouped_tcgen05(act, down, y, 1, rows, width, ff, ff, ff, width, experts, width, 0, tile_expert, stream);
    if (rc != FERRIS_OK) return rc;
    const size_t n4 = (size_t)tokens * (width / 4);
    const size_t want4 = (n4 + 255) / 256;
    ferris_launch(moe_combine_kernel<bf16>, dim3((unsigned)(want4 < 148 * 16 ? want4 : 148 * 16)), dim3(256), 0, s, (const float*)y,
                  width, (const int*)pos, weights, h, ldh, tokens, width / 4, top, accumulate,
                  identity_w ? ids : (const int*)nullptr, experts, (const bf16*)x, ldx, identity_w);
    FERRIS_LAUNCH_CHECK();
}

// scored = 0: the `top` largest logits (+ bias), softmax over those.  scored = 1: see the head of this file; `bias` is
// unused, `correction` fp32 [experts] (may be null), with_weights = the experts that have weights (the router outputs
// from there on are identity experts, handed on as the index with_weights), identity_w fp32 [tokens] (the sum of a token's
// identity weights; may be null when with_weights == experts).
FERRIS_API int ferris_moe_router(const void* x, int ldx, int dtype, const void* w, const float* bias, int* ids,
                                 float* weights, int tokens, int width, int experts, int top, int scored,
                                 const float* correction, int groups, int keep, int with_weights, float* identity_w,
                                 void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (experts <= 0 || experts > MOE_MAX_EXPERTS || top <= 0 || top > experts || top > MOE_MAX_TOP || width <= 0)
        FERRIS_REFUSE("router: %d experts (at most %d), %d chosen (at most %d), width %d", experts, MOE_MAX_EXPERTS, top,
                      MOE_MAX_TOP, width);
    if (scored) {
        if (groups <= 0 || experts % groups || keep < 1 || keep > groups || top > keep * (experts / groups))
            FERRIS_REFUSE("router: %d outputs in %d groups of which %d stay, %d chosen", experts, groups, keep, top);
        if (with_weights < 0 || with_weights > experts || (with_weights < experts && !identity_w))
            FERRIS_REFUSE("router: %d of %d outputs have weights", with_weights, experts);
    } else {
        with_weights = experts;
    }
    const bool per_block = tokens <= 148 * 2;  // few tokens: a block each, so that more warps share the work
    const size_t smem = (per_block ? 1 : 4) * (size_t)((width + 3 * experts + 3) & ~3) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(per_block ? tokens : (tokens + 3) / 4), block(128);
    int rc;
#define FERRIS_ROUTER_RUN(T, B)                                                                                          \
    do {                                                                                                                 \
        if ((rc = ferris_allow_dynamic_smem((const void*)moe_router_kernel<T, B>, smem)) != FERRIS_OK) return rc;        \
        ferris_launch(moe_router_kernel<T, B>, grid, block, smem, s, (const T*)x, ldx, (const T*)w, bias, ids, weights,  \
                      tokens, width, experts, top, scored, correction, groups, keep, with_weights, identity_w);          \
    } while (0)
    if (dtype == FERRIS_F32) {
        if (per_block) FERRIS_ROUTER_RUN(float, true); else FERRIS_ROUTER_RUN(float, false);
    } else if (dtype == FERRIS_BF16) {
        if (per_block) FERRIS_ROUTER_RUN(bf16, true); else FERRIS_ROUTER_RUN(bf16, false);
    } else
        FERRIS_REFUSE("router: unknown dtype %d", dtype);
#undef FERRIS_ROUTER_RUN
    FERRIS_LAUNCH_CHECK();
}

// x [tokens, width] rows ldx apart; gate, up: expert e's [ff, width] matrices lie gate_up_stride elements after expert
// e - 1's (two tensors, or the two halves of one [experts, 2 ff, width]); down [experts, width, ff]; ids int32 and
// weights fp32 [tokens, top]; act [tokens x top, ff] (scratch, the activations' type); h fp32 rows ldh apart.
// With y (scratch, fp32 [tokens x top, width]), `experts` and few enough tokens the weights are read once per expert
// (the expert-major kernels for few tokens and the adding pass); the sums are the same bit for bit either way.
FERRIS_API int ferris_moe_experts_token_major(const void* x, int ldx, int dtype, const void* gate, const void* up,
                                              long long gate_up_stride, const void* down, const int* ids,
                                              const float* weights, void* act, float* h,
                                              int ldh, int tokens, int width, int ff, int top, int accumulate,
                                              float* y, int experts, int act_kind, float act_limit,
                                              const float* identity_w, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (experts <= 0) FERRIS_REFUSE("experts: %d experts", experts);
    if (act_kind < 0 || act_kind > 2) FERRIS_REFUSE("experts: unknown activation %d", act_kind);
    if (width <= 0 || ff <= 0 || top <= 0 || top > MOE_MAX_TOP) FERRIS_REFUSE("experts: width %d, ff %d, %d chosen", width, ff, top);
    if (dtype != FERRIS_F32 && dtype != FERRIS_BF16) FERRIS_REFUSE("experts: unknown dtype %d", dtype);
    const size_t few_up = FEW_WARPS * FEW_RING_BYTES + (size_t)MOE_FEW_ROWS * width * sizeof(float);
    const size_t few_down = FEW_WARPS * FEW_RING_BYTES + (size_t)MOE_FEW_ROWS * ff * sizeof(float);
    if (y && experts > 0 && (long long)tokens * top <= MOE_FEW_MAX_PAIRS && tokens * top > 1 && width % 4 == 0 &&
        ldh % 4 == 0 && (((uintptr_t)y | (uintptr_t)h) & 15) == 0 && few_up <= 200 * 1024 && few_down <= 200 * 1024 &&
        experts <= 65535) {
        cudaStream_t s = (cudaStream_t)stream;
        const int pairs = tokens * top, busy = experts < pairs ? experts : pairs;
        // slabs of rows: as large as still fills the SMs a few times over with the experts that can be busy (a block
        // takes its tokens' rows into shared memory once per slab, so small slabs cost reads of their own)
        auto slab_of = [busy](int rows) {
            int slab = 128;
            while (slab > 4 * FEW_WARPS && (long long)busy * ((rows + slab - 1) / slab) < 148 * 4) slab >>= 1;
            return slab;
        };
        const int slab_up = slab_of(ff), slab_down = slab_of(width);
        const dim3 grid_up(experts, (ff + slab_up - 1) / slab_up), grid_down(experts, (width + slab_down - 1) / slab_down);
        if (grid_up.y > 65535 || grid_down.y > 65535) FERRIS_REFUSE("experts: too many slabs");
        int rc;
#define FERRIS_MOE_FEW(T)                                                                                                 \
    do {                                                                                                                  \
        if ((rc = ferris_allow_dynamic_smem((const void*)moe_gate_up_few_kernel<T>, few_up)) != FERRIS_OK) return rc;     \
        if ((rc = ferris_allow_dynamic_smem((const void*)moe_down_few_kernel<T>, few_down)) != FERRIS_OK) return rc;      \
        ferris_launch(moe_gate_up_few_kernel<T>, grid_up, dim3(32 * FEW_WARPS), few_up, s, (const T*)x, ldx, (const T*)gate,         \
                      (const T*)up, (size_t)gate_up_stride, ids, (T*)act, width, ff, pairs, top, slab_up, act_kind,    \
                      act_limit);                                                                                         \
        ferris_launch(moe_down_few_kernel<T>, grid_down, dim3(32 * FEW_WARPS), few_down, s, (const T*)act, (const T*)down, ids, y,   \
                      width, ff, pairs, slab_down);                                                                       \
    } while (0)
        if (dtype == FERRIS_F32)
            FERRIS_MOE_FEW(float);
        else
            FERRIS_MOE_FEW(bf16);
#undef FERRIS_MOE_FEW
        const size_t n4 = (size_t)tokens * (width / 4);
        const size_t want4 = (n4 + 255) / 256;
        const int* skip = identity_w ? ids : (const int*)nullptr;
        if (dtype == FERRIS_F32)
            ferris_launch(moe_combine_kernel<float>, dim3((unsigned)(want4 < 148 * 16 ? want4 : 148 * 16)), dim3(256), 0, s,
                          (const float*)y, width, (const int*)nullptr, weights, h, ldh, tokens, width / 4, top, accumulate,
                          skip, experts, (const float*)x, ldx, identity_w);
        else
            ferris_launch(moe_combine_kernel<bf16>, dim3((unsigned)(want4 < 148 * 16 ? want4 : 148 * 16)), dim3(256), 0, s,
                          (const float*)y, width, (const int*)nullptr, weights, h, ldh, tokens, width / 4, top, accumulate,
                          skip, experts, (const bf16*)x, ldx, identity_w);
        FERRIS_LAUNCH_CHECK();
    }
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
                      (const T*)gate, (const T*)up, (size_t)gate_up_stride, ids, (T*)act, width, ff, top, slab_up,      \
                      experts, act_kind, act_limit);                                                                      \
        ferris_launch(moe_down_kernel<T>, grid_down, dim3(128), smem_down, s, (const T*)act, (const T*)down, ids, weights, \
                      h, ldh, width, ff, top, slab_down, accumulate, experts, (const T*)x, ldx, identity_w);              \
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
