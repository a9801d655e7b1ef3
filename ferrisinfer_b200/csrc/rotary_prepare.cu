// What stands between the q/k product and attention where queries and keys are normed over their whole projection
// and then rotated, and where the keys as projected may serve as the values:
//
//   q <- q / sqrt(mean(q^2) + eps) * wq      the mean over ALL heads' elements of the token at once (wq spans them)
//   k <- k / sqrt(mean(k^2) + eps) * wk      likewise; either norm is skipped when its weight is null
//   values = the third part of the row, or (values_from_keys) k as projected, before the norm
//   the first R elements of every q and k head rotated by the token's position: the pair (u, v), elements
//   (i, i + R/2) of a head ("half") or (2i, 2i + 1) ("interleaved"), becomes (u c - v s, v c + u s) with
//   c = mag cos(pos * freq[i]), s = mag sin(pos * freq[i]); the other elements pass
//   q rewritten in place, k and the values stored into the paged cache.
//
// Rows: [nh d | nkv d | nkv dv unless values_from_keys].  Everything is computed in fp32 (position x frequency as one
// fp32 product, sincosf in full precision); one block per token.
//
// Two kernels.  The paired one (even head sizes and row strides, rows that start on a pair): a token's cosines and
// sines are formed once in shared memory and serve all its heads, both sums of squares come out of one pass and one
// reduction, and every thread loads, norms, rotates and stores two neighbouring elements at a time (in the
// interleaved layout a pair that rotates together is one such load).  The general one takes every other geometry
// element by element.
#include <math.h>
#include <stdint.h>

#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(128) qk_norm_rotary_cache_write_kernel(
    T* qkv, int ld, const int* __restrict__ positions, const int* __restrict__ slot_mapping, T* __restrict__ k_cache,
    T* __restrict__ v_cache, int nh, int nkv, int d, int dv, int page_size, const float* __restrict__ q_weight,
    const float* __restrict__ k_weight, float eps, const float* __restrict__ freq, int rotary, int interleaved, float mag,
    int values_from_keys, int write_kv) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = positions[t];
    T* row = qkv + (size_t)t * ld;
    const int nq = nh * d, nk = nkv * d;
    float inv_q = 1.0f, inv_k = 1.0f;
    if (q_weight) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < nq; i += blockDim.x) {
            const float v = to_float(row[i]);
            ss = fmaf(v, v, ss);
        }
        inv_q = 1.0f / sqrtf(block_sum(ss, scratch) / (float)nq + eps);
    }
    if (k_weight) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < nk; i += blockDim.x) {
            const float v = to_float(row[nq + i]);
            ss = fmaf(v, v, ss);
        }
        inv_k = 1.0f / sqrtf(block_sum(ss, scratch) / (float)nk + eps);
    }
    const int slot = write_kv ? slot_mapping[t] : -1;
    const int page = slot >= 0 ? slot / page_size : 0;
    const int in_page = slot >= 0 ? slot % page_size : 0;
    if (slot >= 0) {  // the values first: where they are the keys as projected, before anything touches those
        const T* vrow = values_from_keys ? row + nq : row + nq + nk;
        for (int e = threadIdx.x; e < nkv * dv; e += blockDim.x) {
            const int h = e / dv, i = e % dv;
            v_cache[(((size_t)page * nkv + h) * page_size + in_page) * dv + i] = vrow[e];
        }
    }
    const int half = rotary >> 1;
    const int last = slot >= 0 ? nq + nk : nq;  // without a cache to write, the keys are left alone
    for (int e = threadIdx.x; e < last; e += blockDim.x) {
        const bool is_q = e < nq;
        const int h = is_q ? e / d : (e - nq) / d;
        const int i = is_q ? e % d : (e - nq) % d;
        const float inv = is_q ? inv_q : inv_k;
        const float* w = is_q ? q_weight : k_weight;
        const int col = is_q ? e : e - nq;  // the element's place in its projection, where its norm weight lies
        T* dst = is_q ? row + e - i : k_cache + (((size_t)page * nkv + h) * page_size + in_page) * d;
        if (i >= rotary) {
            const float x = to_float(row[e]);
            dst[i] = from_float<T>(w ? (x * inv) * w[col] : x);
            continue;
        }
        // the first member of a pair works for both
        int partner, f;
        if (interleaved) {
            if (i & 1) continue;
            partner = 1, f = i >> 1;
        } else {
            if (i >= half) continue;
            partner = half, f = i;
        }
        float u = to_float(row[e]), v = to_float(row[e + partner]);
        if (w) u = (u * inv) * w[col], v = (v * inv) * w[col + partner];
        float s, c;
        sincosf((float)pos * freq[f], &s, &c);
        s *= mag, c *= mag;
        dst[i] = from_float<T>(u * c - v * s);
        dst[i + partner] = from_float<T>(v * c + u * s);
    }
}

__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const bf16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ void store2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store2(bf16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// Two sums over a block at once; every thread gets both.  `scratch` holds 66 floats.
__device__ __forceinline__ float2 block_sum2(float a, float b, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    a = warp_sum(a), b = warp_sum(b);
    if (lane == 0) scratch[warp] = a, scratch[32 + warp] = b;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    if (warp == 0) {
        float x = lane < nwarps ? scratch[lane] : 0.0f, y = lane < nwarps ? scratch[32 + lane] : 0.0f;
        x = warp_sum(x), y = warp_sum(y);
        if (lane == 0) scratch[64] = x, scratch[65] = y;
    }
    __syncthreads();
    return make_float2(scratch[64], scratch[65]);
}

// d, dv, ld, nq, nk even; rows and caches start on a pair of elements.  Dynamic shared memory: `rotary` floats (the
// token's cosines, then its sines, both times mag).
template <typename T, bool INTERLEAVED>
__global__ void __launch_bounds__(256) qk_norm_rotary_cache_write_paired_kernel(
    T* qkv, int ld, const int* __restrict__ positions, const int* __restrict__ slot_mapping, T* __restrict__ k_cache,
    T* __restrict__ v_cache, int nh, int nkv, int d, int dv, int page_size, const float* __restrict__ q_weight,
    const float* __restrict__ k_weight, float eps, const float* __restrict__ freq, int rotary, float mag,
    int values_from_keys, int write_kv) {
    extern __shared__ float cs[];
    __shared__ float scratch[66];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int half = rotary >> 1;
    const int pos = positions[t];
    for (int f = threadIdx.x; f < half; f += blockDim.x) {
        float s, c;
        sincosf((float)pos * freq[f], &s, &c);
        cs[f] = c * mag, cs[half + f] = s * mag;
    }
    const int slot = write_kv ? slot_mapping[t] : -1;
    T* row = qkv + (size_t)t * ld;
    const int nq = nh * d, nk = nkv * d;
    float sq = 0.0f, sk = 0.0f;
    if (q_weight)
        for (int e = 2 * threadIdx.x; e < nq; e += 2 * blockDim.x) {
            const float2 v = load2(row + e);
            sq = fmaf(v.x, v.x, sq), sq = fmaf(v.y, v.y, sq);
        }
    if (k_weight)
        for (int e = 2 * threadIdx.x; e < nk; e += 2 * blockDim.x) {
            const float2 v = load2(row + nq + e);
            sk = fmaf(v.x, v.x, sk), sk = fmaf(v.y, v.y, sk);
        }
    const float2 sums = block_sum2(sq, sk, scratch);  // also: the table is written
    const float inv_q = q_weight ? 1.0f / sqrtf(sums.x / (float)nq + eps) : 1.0f;
    const float inv_k = k_weight ? 1.0f / sqrtf(sums.y / (float)nk + eps) : 1.0f;
    const int page = slot >= 0 ? slot / page_size : 0;
    const int in_page = slot >= 0 ? slot % page_size : 0;
    if (slot >= 0) {
        const T* vrow = values_from_keys ? row + nq : row + nq + nk;
        for (int e = 2 * threadIdx.x; e < nkv * dv; e += 2 * blockDim.x) {
            const int h = e / dv, i = e - h * dv;
            const float2 v = load2(vrow + e);
            store2(v_cache + (((size_t)page * nkv + h) * page_size + in_page) * dv + i, v.x, v.y);
        }
    }
    const int last = slot >= 0 ? nq + nk : nq;
    const int per_head = d >> 1;  // items of a head: its rotating pairs, then its other elements two by two
    for (int item = threadIdx.x; item < (last >> 1); item += blockDim.x) {
        const int head = item / per_head, j = item - head * per_head;
        const bool is_q = head < nh;
        const int h = is_q ? head : head - nh;
        const float inv = is_q ? inv_q : inv_k;
        const float* w = is_q ? q_weight : k_weight;
        const T* src = row + (size_t)head * d;
        const float* wh = w ? w + (size_t)h * d : nullptr;
        T* dst = is_q ? row + (size_t)head * d : k_cache + (((size_t)page * nkv + h) * page_size + in_page) * d;
        if (j >= half) {  // two elements that pass
            const int i = rotary + 2 * (j - half);
            float2 x = load2(src + i);
            if (w) x.x = (x.x * inv) * wh[i], x.y = (x.y * inv) * wh[i + 1];
            store2(dst + i, x.x, x.y);
            continue;
        }
        const float c = cs[j], s = cs[half + j];
        if (INTERLEAVED) {
            const int i = 2 * j;
            float2 x = load2(src + i);
            if (w) x.x = (x.x * inv) * wh[i], x.y = (x.y * inv) * wh[i + 1];
            store2(dst + i, x.x * c - x.y * s, x.y * c + x.x * s);
        } else {
            float u = to_float(src[j]), v = to_float(src[j + half]);
            if (w) u = (u * inv) * wh[j], v = (v * inv) * wh[j + half];
            dst[j] = from_float<T>(u * c - v * s);
            dst[j + half] = from_float<T>(v * c + u * s);
        }
    }
}

// The norm per HEAD: every q and k head divided by the root mean square of its own d elements and multiplied by a
// weight of d numbers that all heads share (wq for queries, wk for keys; null: that side is not normed), then rotated
// and stored as above.  A warp per head: its lanes sum the head's squares, then norm, rotate and store it; the values
// are copied by the whole block.  With freq_lo (what the 32-bit frequencies lack of their 64-bit values) the angle
// position x frequency keeps the digits that one 32-bit product rounds away: the product's own rounding error comes
// from an FMA, the frequency's from freq_lo, and the small sum e of the two enters as sin(a + e) = sin a + e cos a,
// cos(a + e) = cos a - e sin a.  At position 1,000 a 32-bit angle is off by up to 6e-5 rad, which shows in 32-bit logits.
template <typename T>
__global__ void __launch_bounds__(256) qk_head_norm_rotary_cache_write_kernel(
    T* qkv, int ld, const int* __restrict__ positions, const int* __restrict__ slot_mapping, T* __restrict__ k_cache,
    T* __restrict__ v_cache, int nh, int nkv, int d, int dv, int page_size, const float* __restrict__ q_weight,
    const float* __restrict__ k_weight, float eps, const float* __restrict__ freq, int rotary, int interleaved, float mag,
    int write_kv, const float* __restrict__ freq_lo) {
    extern __shared__ float cs[];  // the token's cosines, then its sines, both times mag
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rotary >> 1;
    for (int f = threadIdx.x; f < half; f += blockDim.x) {
        const float p = (float)pos, hi = freq[f];
        const float angle = p * hi;
        float s, c;
        sincosf(angle, &s, &c);
        if (freq_lo) {
            const float e = fmaf(p, hi, -angle) + p * freq_lo[f];
            const float s0 = s;
            s = fmaf(e, c, s), c = fmaf(-e, s0, c);
        }
        cs[f] = c * mag, cs[half + f] = s * mag;
    }
    __syncthreads();
    T* row = qkv + (size_t)t * ld;
    const int nq = nh * d, nk = nkv * d;
    const int slot = write_kv ? slot_mapping[t] : -1;
    const int page = slot >= 0 ? slot / page_size : 0;
    const int in_page = slot >= 0 ? slot % page_size : 0;
    if (slot >= 0) {
        const T* vrow = row + nq + nk;
        for (int e = threadIdx.x; e < nkv * dv; e += blockDim.x) {
            const int h = e / dv, i = e - h * dv;
            v_cache[(((size_t)page * nkv + h) * page_size + in_page) * dv + i] = vrow[e];
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int heads = slot >= 0 ? nh + nkv : nh;  // without a cache to write, the keys are left alone
    for (int head = warp; head < heads; head += warps) {
        const bool is_q = head < nh;
        const int h = is_q ? head : head - nh;
        const float* w = is_q ? q_weight : k_weight;
        const T* src = row + (size_t)head * d;
        T* dst = is_q ? row + (size_t)head * d : k_cache + (((size_t)page * nkv + h) * page_size + in_page) * d;
        float inv = 1.0f;
        if (w) {
            float ss = 0.0f;
            for (int i = lane; i < d; i += 32) {
                const float x = to_float(src[i]);
                ss = fmaf(x, x, ss);
            }
            inv = 1.0f / sqrtf(warp_sum(ss) / (float)d + eps);  // every lane has read the head before any lane writes it
        }
        for (int j = lane; j < half; j += 32) {
            const int i0 = interleaved ? 2 * j : j, i1 = interleaved ? 2 * j + 1 : j + half;
            float u = to_float(src[i0]), v = to_float(src[i1]);
            if (w) u = (u * inv) * w[i0], v = (v * inv) * w[i1];
            const float c = cs[j], s = cs[half + j];
            dst[i0] = from_float<T>(u * c - v * s);
            dst[i1] = from_float<T>(v * c + u * s);
        }
        for (int i = rotary + lane; i < d; i += 32) {
            const float x = to_float(src[i]);
            dst[i] = from_float<T>(w ? (x * inv) * w[i] : x);
        }
    }
}

}  // namespace

FERRIS_API int ferris_qk_norm_rotary_cache_write(void* qkv, int ld, int dtype, const int* positions,
                                                 const int* slot_mapping, void* k_cache, void* v_cache, int tokens, int nh,
                                                 int nkv, int d, int dv, int page_size, const float* q_weight,
                                                 const float* k_weight, float eps, const float* freq, int rotary,
                                                 int interleaved, float mag, int values_from_keys, int write_kv,
                                                 void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (nh <= 0 || nkv <= 0 || d <= 0 || dv <= 0 || page_size <= 0)
        FERRIS_REFUSE("qk norm + rotation: nh=%d nkv=%d d=%d dv=%d page_size=%d", nh, nkv, d, dv, page_size);
    if (rotary < 0 || rotary > d || (rotary & 1) || (rotary > 0 && !freq))
        FERRIS_REFUSE("qk norm + rotation: %d rotated elements of heads of %d", rotary, d);
    if (values_from_keys && dv != d) FERRIS_REFUSE("qk norm + rotation: keys of %d cannot serve as values of %d", d, dv);
    if (ld < (nh + nkv) * d + (values_from_keys ? 0 : nkv * dv)) FERRIS_REFUSE("qk norm + rotation: rows of %d are too short", ld);
    if (write_kv && (!slot_mapping || !k_cache || !v_cache)) FERRIS_REFUSE("qk norm + rotation: no cache to write");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t elem = dtype == FERRIS_F32 ? 4 : 2;
    const bool paired = !((d | dv | ld) & 1) && (uintptr_t)qkv % (2 * elem) == 0 && (uintptr_t)k_cache % (2 * elem) == 0 &&
                        (uintptr_t)v_cache % (2 * elem) == 0 && ((uintptr_t)q_weight | (uintptr_t)k_weight) % 8 == 0 &&
                        (dtype == FERRIS_F32 || dtype == FERRIS_BF16);
    if (paired) {
        const size_t smem = (size_t)rotary * sizeof(float);
#define FERRIS_PAIRED(T, I)                                                                                              \
    ferris_launch(qk_norm_rotary_cache_write_paired_kernel<T, I>, dim3(tokens), dim3(256), smem, s, (T*)qkv, ld, positions, \
                  slot_mapping, (T*)k_cache, (T*)v_cache, nh, nkv, d, dv, page_size, q_weight, k_weight, eps, freq, rotary,  \
                  mag, values_from_keys, write_kv)
        if (dtype == FERRIS_F32) {
            if (interleaved) FERRIS_PAIRED(float, true); else FERRIS_PAIRED(float, false);
        } else {
            if (interleaved) FERRIS_PAIRED(bf16, true); else FERRIS_PAIRED(bf16, false);
        }
#undef FERRIS_PAIRED
        FERRIS_LAUNCH_CHECK();
    }
    if (dtype == FERRIS_F32)
        ferris_launch(qk_norm_rotary_cache_write_kernel<float>, dim3(tokens), dim3(128), 0, s, (float*)qkv, ld, positions,
                      slot_mapping, (float*)k_cache, (float*)v_cache, nh, nkv, d, dv, page_size, q_weight, k_weight, eps,
                      freq, rotary, interleaved, mag, values_from_keys, write_kv);
    else if (dtype == FERRIS_BF16)
        ferris_launch(qk_norm_rotary_cache_write_kernel<bf16>, dim3(tokens), dim3(128), 0, s, (bf16*)qkv, ld, positions,
                      slot_mapping, (bf16*)k_cache, (bf16*)v_cache, nh, nkv, d, dv, page_size, q_weight, k_weight, eps,
                      freq, rotary, interleaved, mag, values_from_keys, write_kv);
    else
        FERRIS_REFUSE("qk norm + rotation: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}

// As above with the norm taken per head: q_weight, k_weight fp32 [d] (shared by the heads; null: no norm on that side).
// freq_lo (may be null): fp32 [rotary / 2], the 64-bit frequencies minus their 32-bit roundings.
FERRIS_API int ferris_qk_head_norm_rotary_cache_write(void* qkv, int ld, int dtype, const int* positions,
                                                      const int* slot_mapping, void* k_cache, void* v_cache, int tokens,
                                                      int nh, int nkv, int d, int dv, int page_size, const float* q_weight,
                                                      const float* k_weight, float eps, const float* freq, int rotary,
                                                      int interleaved, float mag, int write_kv, const float* freq_lo,
                                                      void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (nh <= 0 || nkv <= 0 || d <= 0 || dv <= 0 || page_size <= 0)
        FERRIS_REFUSE("head norm + rotation: nh=%d nkv=%d d=%d dv=%d page_size=%d", nh, nkv, d, dv, page_size);
    if (rotary < 0 || rotary > d || (rotary & 1) || (rotary > 0 && !freq))
        FERRIS_REFUSE("head norm + rotation: %d rotated elements of heads of %d", rotary, d);
    if (ld < (nh + nkv) * d + nkv * dv) FERRIS_REFUSE("head norm + rotation: rows of %d are too short", ld);
    if (write_kv && (!slot_mapping || !k_cache || !v_cache)) FERRIS_REFUSE("head norm + rotation: no cache to write");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)(rotary > 0 ? rotary : 1) * sizeof(float);
    const int threads = (nh + nkv) >= 8 ? 256 : 128;
    if (dtype == FERRIS_F32)
        ferris_launch(qk_head_norm_rotary_cache_write_kernel<float>, dim3(tokens), dim3(threads), smem, s, (float*)qkv, ld,
                      positions, slot_mapping, (float*)k_cache, (float*)v_cache, nh, nkv, d, dv, page_size, q_weight, k_weight,
                      eps, freq, rotary, interleaved, mag, write_kv, freq_lo);
    else if (dtype == FERRIS_BF16)
        ferris_launch(qk_head_norm_rotary_cache_write_kernel<bf16>, dim3(tokens), dim3(threads), smem, s, (bf16*)qkv, ld,
                      positions, slot_mapping, (bf16*)k_cache, (bf16*)v_cache, nh, nkv, d, dv, page_size, q_weight, k_weight, eps,
                      freq, rotary, interleaved, mag, write_kv, freq_lo);
    else
        FERRIS_REFUSE("head norm + rotation: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}
