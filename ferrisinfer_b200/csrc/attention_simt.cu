// Attention over the paged cache, general form: any head size up to 512 (the values' may differ
// from the queries' and keys'), any page size, any number of heads and groups, an optional window;
// fp32 arithmetic throughout whatever the storage type.  One block per (token, query head); the warps of a block split the keys and keep
// a running maximum, sum and weighted value sum each, merged at the end.
//
//   query head hq uses kv head hq / (nh / nkv); s_j = (q . k_j) * scale; the query at absolute
//   position P attends keys lo..P, lo = 0, P - window + 1 or (a negative `window`: a chunk of that many positions)
//   the start of P's chunk; softmax over them; out = sum w_j v_j.
//   With `slopes` (one per query head; a position encoding that acts on the scores, not on q and k):
//   s_j += slopes[hq] * (j - P), a penalty linear in the distance.
// (crates/ferrisinfer-kernel/src/cpu/attention.rs:729-781, 1125-1155: streaming softmax with a
// running maximum, which this kernel keeps per warp).  The step's own keys are already in the
// cache when this runs, so prompts, portions of prompts and single decoded tokens are one case.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int ATT_THREADS = 128;
constexpr int ATT_WARPS = ATT_THREADS / 32;
constexpr int MAX_PER_LANE = 16;  // head size up to 512 (the forms below this one: up to 256)

// What else enters a score and the softmax, per query head (any pointer may be null):
//   slopes:        s_j += slopes[h] * (j - P), a penalty linear in the distance;
//   log_r1, log_r2: s_j -= log_r1[h] * ln(1 + log_r2[h] * (P - j)), a penalty that grows with the distance's logarithm;
//   sink:          the softmax's denominator also holds exp(sink[h]): a weight that belongs to no key and no value.
// v_stride: elements between the value rows of consecutive cache rows (0: dv).  With the key cache given as the
// value cache too and v_stride = d, a value is the first dv elements of its key (keys that carry their value).
struct ScoreTerms {
    const float* slopes;
    const float* log_r1;
    const float* log_r2;
    const float* sink;
    int v_stride;
};
struct HeadTerms {
    int kind;  // 0: nothing, 1: slope, 2: logarithm
    float a, b;
};
__device__ __forceinline__ HeadTerms head_terms(const ScoreTerms& st, int h) {
    HeadTerms t = {0, 0.0f, 0.0f};
    if (st.slopes) t.kind = 1, t.a = st.slopes[h];
    if (st.log_r1) t.kind = 2, t.a = st.log_r1[h], t.b = st.log_r2[h];
    return t;
}
// the score of the key at j for the query at P, from the scaled product
__device__ __forceinline__ float with_terms(float s, const HeadTerms& t, int j, int P) {
    if (t.kind == 1) return fmaf(t.a, (float)(j - P), s);
    if (t.kind == 2) return s - t.a * log1pf(t.b * (float)(P - j));
    return s;
}
// The first key that the query at position P sees.  window > 0: the last `window` keys, itself included; window < 0:
// the keys of its own chunk, positions being counted off in chunks of -window from 0; 0: every key.
__device__ __forceinline__ int first_key(int P, int window) {
    if (window > 0) return P - window + 1 > 0 ? P - window + 1 : 0;
    if (window < 0) return P - P % (-window);
    return 0;
}
// the sink's share of the denominator, relative to the maximum mm of the keys' scores
__device__ __forceinline__ float sink_share(const ScoreTerms& st, int h, float mm) { return st.sink ? expf(st.sink[h] - mm) : 0.0f; }

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS)
    paged_attention_simt_kernel(const T* q, int ldq, T* __restrict__ out, int ldo, const T* k_cache, const T* v_cache,
                                const int* __restrict__ block_tables, int max_blocks,
                                const int* __restrict__ token_seq, const int* __restrict__ positions, int nh,
                                int nkv, int d, int dv, int page_size, int window, float scale,
                                const ScoreTerms st) {
    extern __shared__ float smem[];  // per warp: m, z, acc[dv]
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x, hq = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hk = hq / (nh / nkv);
    const int seq = token_seq[t];
    const int P = positions[t];
    const int lo = first_key(P, window);
    const int* table = block_tables + (size_t)seq * max_blocks;
    const HeadTerms ht = head_terms(st, hq);
    const size_t vs = st.v_stride ? st.v_stride : dv;

    float qv[MAX_PER_LANE], acc[MAX_PER_LANE];
    const T* qrow = q + (size_t)t * ldq + (size_t)hq * d;
#pragma unroll
    for (int r = 0; r < MAX_PER_LANE; ++r) {
        const int i = lane + 32 * r;
        qv[r] = i < d ? to_float(qrow[i]) : 0.0f;
        acc[r] = 0.0f;
    }
    float m = -INFINITY, z = 0.0f;
    for (int j = lo + warp; j <= P; j += ATT_WARPS) {
        const int page = table[j / page_size];
        if (page < 0) continue;  // a hole in the table: never reached for keys inside the window
        const size_t row = ((size_t)page * nkv + hk) * page_size + (j % page_size);
        const size_t base = row * d, vbase = row * vs;
        float dot = 0.0f;
#pragma unroll
        for (int r = 0; r < MAX_PER_LANE; ++r) {
            const int i = lane + 32 * r;
            if (i < d) dot = fmaf(qv[r], to_float(k_cache[base + i]), dot);
        }
        const float s = with_terms(warp_sum(dot) * scale, ht, j, P);
        float wgt;
        if (s > m) {
            const float rescale = expf(m - s);  // exp(-inf) = 0 on the first key
#pragma unroll
            for (int r = 0; r < MAX_PER_LANE; ++r) acc[r] *= rescale;
            z = z * rescale + 1.0f;
            m = s;
            wgt = 1.0f;
        } else {
            wgt = expf(s - m);
            z += wgt;
        }
#pragma unroll
        for (int r = 0; r < MAX_PER_LANE; ++r) {
            const int i = lane + 32 * r;
            if (i < dv) acc[r] = fmaf(wgt, to_float(v_cache[vbase + i]), acc[r]);
        }
    }
    float* mine = smem + warp * (dv + 2);
    if (lane == 0) {
        mine[0] = m;
        mine[1] = z;
    }
#pragma unroll
    for (int r = 0; r < MAX_PER_LANE; ++r) {
        const int i = lane + 32 * r;
        if (i < dv) mine[2 + i] = acc[r];
    }
    __syncthreads();
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) mm = fmaxf(mm, smem[w * (dv + 2)]);
    float zz = 0.0f;
    float f[ATT_WARPS];
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
        const float mw = smem[w * (dv + 2)];
        f[w] = mw == -INFINITY ? 0.0f : expf(mw - mm);
        zz += smem[w * (dv + 2) + 1] * f[w];
    }
    zz += sink_share(st, hq, mm);
    const float inv = 1.0f / zz;
    T* orow = out + (size_t)t * ldo + (size_t)hq * dv;
    for (int i = threadIdx.x; i < dv; i += ATT_THREADS) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) o += smem[w * (dv + 2) + 2 + i] * f[w];
        orow[i] = from_float<T>(o * inv);
    }
}


// ---------------------------------------------------------------------------------------------
// The same attention for head sizes that are multiples of eight: EIGHT lanes share a key, so a warp has four keys
// in flight (a block sixteen, two each where registers allow), and every lane reads its eighth of a key or value
// row with the widest loads its size allows (16 bytes at head sizes that are multiples of 64 in bf16).  The dot
// product is summed over the eight lanes with three shuffles; each group of eight keeps a running maximum, sum
// and weighted value sum of its own over its keys lo + g, lo + g + 16, ...; the sixteen groups are merged at the end
// as the four warps are in the kernel above.  Scores, weights and sums are fp32.
// ---------------------------------------------------------------------------------------------
constexpr int AL_THREADS = 128;
constexpr int AL_GROUPS = AL_THREADS / 8;

template <int MAXC>
__device__ __forceinline__ void load_chunk(const float* p, int n, float (&o)[MAXC]) {
    if ((n & 3) == 0) {
#pragma unroll
        for (int i = 0; i < MAXC; i += 4)
            if (i < n) {
                const float4 u = *reinterpret_cast<const float4*>(p + i);
                o[i] = u.x, o[i + 1] = u.y, o[i + 2] = u.z, o[i + 3] = u.w;
            }
    } else {
#pragma unroll
        for (int i = 0; i < MAXC; ++i)
            if (i < n) o[i] = p[i];
    }
}

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

template <int MAXC>
__device__ __forceinline__ void load_chunk(const bf16* p, int n, float (&o)[MAXC]) {
    if ((n & 7) == 0) {
#pragma unroll
        for (int i = 0; i < MAXC; i += 8)
            if (i < n) {
                const uint4 u = *reinterpret_cast<const uint4*>(p + i);
                o[i] = bf16_lo(u.x), o[i + 1] = bf16_hi(u.x), o[i + 2] = bf16_lo(u.y), o[i + 3] = bf16_hi(u.y);
                o[i + 4] = bf16_lo(u.z), o[i + 5] = bf16_hi(u.z), o[i + 6] = bf16_lo(u.w), o[i + 7] = bf16_hi(u.w);
            }
    } else if ((n & 3) == 0) {
#pragma unroll
        for (int i = 0; i < MAXC; i += 4)
            if (i < n) {
                const uint2 u = *reinterpret_cast<const uint2*>(p + i);
                o[i] = bf16_lo(u.x), o[i + 1] = bf16_hi(u.x), o[i + 2] = bf16_lo(u.y), o[i + 3] = bf16_hi(u.y);
            }
    } else if ((n & 1) == 0) {
#pragma unroll
        for (int i = 0; i < MAXC; i += 2)
            if (i < n) {
                const uint32_t u = *reinterpret_cast<const uint32_t*>(p + i);
                o[i] = bf16_lo(u), o[i + 1] = bf16_hi(u);
            }
    } else {
#pragma unroll
        for (int i = 0; i < MAXC; ++i)
            if (i < n) o[i] = __bfloat162float(p[i]);
    }
}

// MAXC: most elements of a head that one lane holds (d, dv <= 8 * MAXC).  U: keys of a group in flight together.
template <typename T, int MAXC, int U>
__global__ void __launch_bounds__(AL_THREADS)
    paged_attention_lanes_kernel(const T* q, int ldq, T* __restrict__ out, int ldo, const T* k_cache, const T* v_cache,
                                 const int* __restrict__ block_tables, int max_blocks,
                                 const int* __restrict__ token_seq, const int* __restrict__ positions, int nh, int nkv,
                                 int d, int dv, int page_size, int window, float scale,
                                 const ScoreTerms st) {
    extern __shared__ float smem[];  // per group: m, z, acc[dv]
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x, hq = blockIdx.y;
    const int sub = threadIdx.x & 7, grp = threadIdx.x >> 3;
    const int hk = hq / (nh / nkv);
    const int seq = token_seq[t];
    const int P = positions[t];
    const int lo = first_key(P, window);
    const int* table = block_tables + (size_t)seq * max_blocks;
    const HeadTerms ht = head_terms(st, hq);
    const size_t vs = st.v_stride ? st.v_stride : dv;
    const int ch = d >> 3, cv = dv >> 3;
    const int pshift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;

    float qv[MAXC], acc[MAXC];
#pragma unroll
    for (int i = 0; i < MAXC; ++i) qv[i] = 0.0f, acc[i] = 0.0f;
    load_chunk<MAXC>(q + (size_t)t * ldq + (size_t)hq * d + sub * ch, ch, qv);
    float m = -INFINITY, z = 0.0f;
    const int rounds = (P - lo + AL_GROUPS * U) / (AL_GROUPS * U);  // every lane of a warp makes as many: the shuffles need all
    for (int it = 0; it < rounds; ++it) {
        float kk[U][MAXC], vv[U][MAXC];
        bool ok[U];
        int jj[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = lo + (it * U + u) * AL_GROUPS + grp;
            jj[u] = j;
            int page = -1;
            if (j <= P) page = table[pshift >= 0 ? (j >> pshift) : (j / page_size)];
            ok[u] = page >= 0;  // beyond the last key, or a hole in the table (never for keys inside the window)
            const int in_page = pshift >= 0 ? (j & (page_size - 1)) : (j % page_size);
            const size_t row = ((size_t)(ok[u] ? page : 0) * nkv + hk) * page_size + (ok[u] ? in_page : 0);
#pragma unroll
            for (int i = 0; i < MAXC; ++i) kk[u][i] = 0.0f, vv[u][i] = 0.0f;
            if (ok[u]) {
                load_chunk<MAXC>(k_cache + row * d + sub * ch, ch, kk[u]);
                load_chunk<MAXC>(v_cache + row * vs + sub * cv, cv, vv[u]);
            }
        }
        float dot[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float a = 0.0f;
#pragma unroll
            for (int i = 0; i < MAXC; ++i) a = fmaf(qv[i], kk[u][i], a);
            dot[u] = a;
        }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < U; ++u) dot[u] += __shfl_xor_sync(0xffffffffu, dot[u], o);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (!ok[u]) continue;
            const float s = with_terms(dot[u] * scale, ht, jj[u], P);
            float wgt;
            if (s > m) {
                const float rescale = expf(m - s);  // exp(-inf) = 0 on the first key
#pragma unroll
                for (int i = 0; i < MAXC; ++i) acc[i] *= rescale;
                z = z * rescale + 1.0f;
                m = s;
                wgt = 1.0f;
            } else {
                wgt = expf(s - m);
                z += wgt;
            }
#pragma unroll
            for (int i = 0; i < MAXC; ++i) acc[i] = fmaf(wgt, vv[u][i], acc[i]);
        }
    }
    float* mine = smem + grp * (dv + 2);
    if (sub == 0) {
        mine[0] = m;
        mine[1] = z;
    }
#pragma unroll
    for (int i = 0; i < MAXC; ++i)
        if (i < cv) mine[2 + sub * cv + i] = acc[i];
    __syncthreads();
    float mm = -INFINITY;
    for (int g = 0; g < AL_GROUPS; ++g) mm = fmaxf(mm, smem[g * (dv + 2)]);
    float zz = 0.0f;
    float f[AL_GROUPS];
#pragma unroll
    for (int g = 0; g < AL_GROUPS; ++g) {
        const float mg = smem[g * (dv + 2)];
        f[g] = mg == -INFINITY ? 0.0f : expf(mg - mm);
        zz += smem[g * (dv + 2) + 1] * f[g];
    }
    zz += sink_share(st, hq, mm);
    const float inv = 1.0f / zz;
    T* orow = out + (size_t)t * ldo + (size_t)hq * dv;
    for (int i = threadIdx.x; i < dv; i += AL_THREADS) {
        float o = 0.0f;
#pragma unroll
        for (int g = 0; g < AL_GROUPS; ++g) o += smem[g * (dv + 2) + 2 + i] * f[g];
        orow[i] = from_float<T>(o * inv);
    }
}

// Single tokens where several query heads share a kv head: a block takes G of those heads at once, SIXTEEN lanes share
// a key and hold a sixteenth of it, so a key and its value are read, and widened to fp32, once for the G heads, and
// each group of sixteen keeps U keys in flight.  What bounds a step of single tokens is the bytes in flight per SM.
constexpr int AG_THREADS = 128;
constexpr int AG_GROUPS = AG_THREADS / 16;

template <typename T, int MAXC, int G, int U>
__global__ void __launch_bounds__(AG_THREADS)
    paged_attention_shared_kernel(const T* q, int ldq, T* __restrict__ out, int ldo, const T* k_cache, const T* v_cache,
                                  const int* __restrict__ block_tables, int max_blocks,
                                  const int* __restrict__ token_seq, const int* __restrict__ positions, int nh, int nkv,
                                  int d, int dv, int page_size, int window, float scale,
                                  const ScoreTerms st, int splits, float* __restrict__ partial) {
    extern __shared__ float smem[];  // per group and head: m, z, acc[dv]
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x, h0 = blockIdx.y * G;  // query heads h0 .. h0 + G - 1, all of one kv head
    const int split = blockIdx.z;
    const int sub = threadIdx.x & 15, grp = threadIdx.x >> 4;
    const int hk = h0 / (nh / nkv);
    const int seq = token_seq[t];
    const int P = positions[t];
    const int lo = first_key(P, window);
    const int* table = block_tables + (size_t)seq * max_blocks;
    const int ch = d >> 4, cv = dv >> 4;
    const size_t vs = st.v_stride ? st.v_stride : dv;
    const int pshift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;

    float qv[G][MAXC], acc[G][MAXC], m[G], z[G];
    HeadTerms ht[G];
#pragma unroll
    for (int a = 0; a < G; ++a) {
#pragma unroll
        for (int i = 0; i < MAXC; ++i) qv[a][i] = 0.0f, acc[a][i] = 0.0f;
        load_chunk<MAXC>(q + (size_t)t * ldq + (size_t)(h0 + a) * d + sub * ch, ch, qv[a]);
        m[a] = -INFINITY, z[a] = 0.0f;
        ht[a] = head_terms(st, h0 + a);
    }
    // the block's share of the keys lo .. P: with several splits, a run of `span` keys each
    const int span = (P - lo + splits) / splits;
    const int first = lo + split * span;
    const int lastk = min(P, first + span - 1);
    const int rounds = lastk >= first ? (lastk - first + AG_GROUPS * U) / (AG_GROUPS * U) : 0;
    for (int it = 0; it < rounds; ++it) {
        float kk[U][MAXC], vv[U][MAXC];
        bool ok[U];
        int jj[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = first + (it * U + u) * AG_GROUPS + grp;
            jj[u] = j;
            int page = -1;
            if (j <= lastk) page = table[pshift >= 0 ? (j >> pshift) : (j / page_size)];
            ok[u] = page >= 0;
            const int in_page = pshift >= 0 ? (j & (page_size - 1)) : (j % page_size);
            const size_t row = ((size_t)(ok[u] ? page : 0) * nkv + hk) * page_size + (ok[u] ? in_page : 0);
#pragma unroll
            for (int i = 0; i < MAXC; ++i) kk[u][i] = 0.0f, vv[u][i] = 0.0f;
            if (ok[u]) {
                load_chunk<MAXC>(k_cache + row * d + sub * ch, ch, kk[u]);
                load_chunk<MAXC>(v_cache + row * vs + sub * cv, cv, vv[u]);
            }
        }
        float dot[U][G];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int a = 0; a < G; ++a) {
                float x = 0.0f;
#pragma unroll
                for (int i = 0; i < MAXC; ++i) x = fmaf(qv[a][i], kk[u][i], x);
                dot[u][a] = x;
            }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int a = 0; a < G; ++a) dot[u][a] += __shfl_xor_sync(0xffffffffu, dot[u][a], o);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (!ok[u]) continue;
#pragma unroll
            for (int a = 0; a < G; ++a) {
                const float s = with_terms(dot[u][a] * scale, ht[a], jj[u], P);
                float wgt;
                if (s > m[a]) {
                    const float rescale = expf(m[a] - s);
#pragma unroll
                    for (int i = 0; i < MAXC; ++i) acc[a][i] *= rescale;
                    z[a] = z[a] * rescale + 1.0f;
                    m[a] = s;
                    wgt = 1.0f;
                } else {
                    wgt = expf(s - m[a]);
                    z[a] += wgt;
                }
#pragma unroll
                for (int i = 0; i < MAXC; ++i) acc[a][i] = fmaf(wgt, vv[u][i], acc[a][i]);
            }
        }
    }
    const int stride = dv + 2;
#pragma unroll
    for (int a = 0; a < G; ++a) {
        float* mine = smem + (size_t)(grp * G + a) * stride;
        if (sub == 0) {
            mine[0] = m[a];
            mine[1] = z[a];
        }
#pragma unroll
        for (int i = 0; i < MAXC; ++i)
            if (i < cv) mine[2 + sub * cv + i] = acc[a][i];
    }
    __syncthreads();
    for (int w = threadIdx.x; w < G * dv; w += AG_THREADS) {
        const int a = w / dv, i = w % dv;
        float mm = -INFINITY;
        for (int g2 = 0; g2 < AG_GROUPS; ++g2) mm = fmaxf(mm, smem[(size_t)(g2 * G + a) * stride]);
        float zz = 0.0f, o = 0.0f;
        for (int g2 = 0; g2 < AG_GROUPS; ++g2) {
            const float* e = smem + (size_t)(g2 * G + a) * stride;
            const float f = e[0] == -INFINITY ? 0.0f : expf(e[0] - mm);
            zz += e[1] * f;
            o += e[2 + i] * f;
        }
        if (splits == 1) {
            zz += sink_share(st, h0 + a, mm);
            out[(size_t)t * ldo + (size_t)(h0 + a) * dv + i] = from_float<T>(o / zz);
        } else {  // the share's maximum, sum and weighted values, for the merge kernel
            float* e = partial + (((size_t)t * nh + h0 + a) * splits + split) * stride;
            if (i == 0) e[0] = mm, e[1] = zz;
            e[2 + i] = o;
        }
    }
}

// out = sum_s o_s e^(m_s - M) / sum_s z_s e^(m_s - M) over the shares of the keys that the kernel above left in `partial`
// ([tokens, heads, splits, 2 + dv]: maximum, sum, weighted values).  A block per (token, head).
template <typename T>
__global__ void __launch_bounds__(128) attention_merge_shares_kernel(const float* partial, T* __restrict__ out, int ldo,
                                                                     int nh, int dv, int splits, const ScoreTerms st) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x, h = blockIdx.y;
    const int stride = dv + 2;
    const float* base = partial + ((size_t)t * nh + h) * splits * stride;
    float mm = -INFINITY;
    for (int s2 = 0; s2 < splits; ++s2) mm = fmaxf(mm, base[(size_t)s2 * stride]);
    float zz = 0.0f;
    for (int s2 = 0; s2 < splits; ++s2) {
        const float ms = base[(size_t)s2 * stride];
        zz += ms == -INFINITY ? 0.0f : base[(size_t)s2 * stride + 1] * expf(ms - mm);
    }
    zz += sink_share(st, h, mm);
    const float inv = 1.0f / zz;
    for (int i = threadIdx.x; i < dv; i += blockDim.x) {
        float o = 0.0f;
        for (int s2 = 0; s2 < splits; ++s2) {
            const float ms = base[(size_t)s2 * stride];
            if (ms != -INFINITY) o += base[(size_t)s2 * stride + 2 + i] * expf(ms - mm);
        }
        out[(size_t)t * ldo + (size_t)h * dv + i] = from_float<T>(o * inv);
    }
}

template <typename T, int G>
void launch_shared(const void* q, int ldq, void* out, int ldo, const void* k_cache, const void* v_cache,
                   const int* block_tables, int max_blocks, const int* token_seq, const int* positions, int tokens, int nh,
                   int nkv, int d, int dv, int page_size, int window, float scale, const ScoreTerms st, int splits,
                   float* partial, cudaStream_t s) {
    const dim3 grid(tokens, nh / G, splits), block(AG_THREADS);
    const size_t smem = (size_t)AG_GROUPS * G * (dv + 2) * sizeof(float);
    const int most = d > dv ? d : dv;
#define FERRIS_AG_LAUNCH(MAXC, U)                                                                                       \
    ferris_launch(paged_attention_shared_kernel<T, MAXC, G, U>, grid, block, smem, s, (const T*)q, ldq, (T*)out, ldo,   \
                  (const T*)k_cache, (const T*)v_cache, block_tables, max_blocks, token_seq, positions, nh, nkv, d, dv,  \
                  page_size, window, scale, st, splits, partial)
    if (most <= 128)
        FERRIS_AG_LAUNCH(8, 4);
    else
        FERRIS_AG_LAUNCH(16, 2);
#undef FERRIS_AG_LAUNCH
    if (splits > 1)
        ferris_launch(attention_merge_shares_kernel<T>, dim3(tokens, nh), dim3(128), 0, s, (const float*)partial, (T*)out,
                      ldo, nh, dv, splits, st);
}

template <typename T>
void launch_lanes(const void* q, int ldq, void* out, int ldo, const void* k_cache, const void* v_cache,
                  const int* block_tables, int max_blocks, const int* token_seq, const int* positions, int tokens, int nh,
                  int nkv, int d, int dv, int page_size, int window, float scale, const ScoreTerms st, cudaStream_t s) {
    const dim3 grid(tokens, nh), block(AL_THREADS);
    const size_t smem = (size_t)AL_GROUPS * (dv + 2) * sizeof(float);
    const int most = d > dv ? d : dv;
#define FERRIS_AL_LAUNCH(MAXC, U)                                                                                      \
    ferris_launch(paged_attention_lanes_kernel<T, MAXC, U>, grid, block, smem, s, (const T*)q, ldq, (T*)out, ldo,      \
                  (const T*)k_cache, (const T*)v_cache, block_tables, max_blocks, token_seq, positions, nh, nkv, d, dv, \
                  page_size, window, scale, st)
    if (most <= 64)
        FERRIS_AL_LAUNCH(8, 2);
    else if (most <= 128)
        FERRIS_AL_LAUNCH(16, 2);
    else
        FERRIS_AL_LAUNCH(32, 1);
#undef FERRIS_AL_LAUNCH
}


// ---------------------------------------------------------------------------------------------
// Portions of prompts: a block takes up to TL_ROWS = 64 query rows that share their keys and values, namely the g query
// heads of one kv head for floor(64 / g) consecutive tokens of the step (rows beyond those stay idle), and walks the keys those tokens see in tiles of 32, which
// it brings into shared memory once for all 64 rows (fp32, a row's 16-byte pieces spread over the banks).  Eight
// lanes share two rows: each forms 2 x 4 scores of a tile from shared memory, the eight exchange the rows' maxima
// and sums by shuffles, write the weights to shared memory and add 2 x (dv / 8) columns of weighted values each.
// Everything is fp32 FMAs: scores, weights and the sums over values.  Tokens of several requests in one tile are taken
// request by request (the other rows masked), so any division of a step is served; a step of single tokens is the
// kernel above's.
// ---------------------------------------------------------------------------------------------
constexpr int TL_ROWS = 64, TL_KEYS = 32, TL_THREADS = 256;

__device__ __forceinline__ void stage_row(const float* src, float* dst, int n, int part, int parts, float mul) {
    for (int v = part; v * 4 < n; v += parts) {
        float4 u = *reinterpret_cast<const float4*>(src + v * 4);
        u.x *= mul, u.y *= mul, u.z *= mul, u.w *= mul;
        *reinterpret_cast<float4*>(dst + v * 4) = u;
    }
}
__device__ __forceinline__ void stage_row(const bf16* src, float* dst, int n, int part, int parts, float mul) {
    for (int v = part; v * 8 < n; v += parts) {
        const uint4 u = *reinterpret_cast<const uint4*>(src + v * 8);
        *reinterpret_cast<float4*>(dst + v * 8) = make_float4(bf16_lo(u.x) * mul, bf16_hi(u.x) * mul, bf16_lo(u.y) * mul, bf16_hi(u.y) * mul);
        *reinterpret_cast<float4*>(dst + v * 8 + 4) = make_float4(bf16_lo(u.z) * mul, bf16_hi(u.z) * mul, bf16_lo(u.w) * mul, bf16_hi(u.w) * mul);
    }
}
__device__ __forceinline__ void zero_row(float* dst, int n, int part, int parts) {
    for (int v = part; v * 4 < n; v += parts) *reinterpret_cast<float4*>(dst + v * 4) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
}

template <typename T, int NC>  // NC: 4-column pieces of the value head that a lane adds up: dv <= 32 * NC
__global__ void __launch_bounds__(TL_THREADS)
    paged_attention_tiled_kernel(const T* q, int ldq, T* __restrict__ out, int ldo, const T* k_cache, const T* v_cache,
                                 const int* __restrict__ block_tables, int max_blocks,
                                 const int* __restrict__ token_seq, const int* __restrict__ positions, int tokens, int nh,
                                 int nkv, int d, int dv, int page_size, int window, float scale,
                                 const ScoreTerms st) {
    extern __shared__ __align__(16) float tl_smem[];
    const int dp = d + 4, dvp = dv + 4;
    float* Qs = tl_smem;                      // [64][d + 4], scaled
    float* Ks = Qs + TL_ROWS * dp;            // [32][d + 4]
    float* Vs = Ks + TL_KEYS * dp;            // [32][dv + 4]
    float* Ps = Vs + TL_KEYS * dvp;           // [64][32 + 1]
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x;
    const int g = nh / nkv, qt = TL_ROWS / g;
    const int hk = blockIdx.y;
    const int t_first = blockIdx.x * qt;
    const int t_end = min(t_first + qt, tokens);
    const int pshift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;

    // the queries, scaled once
    {
        const int row = tid >> 2, part = tid & 3;
        const int t = t_first + row / g;
        float* dst = Qs + row * dp;
        if (t < t_end)
            stage_row(q + (size_t)t * ldq + (size_t)(hk * g + row % g) * d, dst, d, part, 4, scale);
        else
            zero_row(dst, d, part, 4);
    }
    const int ry = tid >> 3, kx = tid & 7;
    const int r0 = 2 * ry;  // this lane's rows: r0 and r0 + 1
    int rt[2], rpos[2], rseq[2];
    HeadTerms rterm[2];
#pragma unroll
    for (int a = 0; a < 2; ++a) {
        rt[a] = t_first + (r0 + a) / g;
        const bool ok = rt[a] < t_end;
        rpos[a] = ok ? positions[rt[a]] : -1;
        rseq[a] = ok ? token_seq[rt[a]] : -1;
        rterm[a] = head_terms(st, hk * g + (r0 + a) % g);
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    float acc[2][NC][4];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[a][c][e] = 0.0f;

    const int seq_first = token_seq[t_first], seq_last = token_seq[t_end - 1];
    int ta = t_first;  // first token of the current request within the tile
    for (int sq = seq_first; sq <= seq_last; ++sq) {
        int tb = ta;  // its last token within the tile
        while (tb + 1 < t_end && token_seq[tb + 1] == sq) ++tb;
        const int pa = positions[ta], pb = positions[tb];
        const int kmin = first_key(pa, window);  // of the first token: no later token of the request sees an earlier key
        const int* table = block_tables + (size_t)sq * max_blocks;
        for (int j0 = kmin & ~(TL_KEYS - 1); j0 <= pb; j0 += TL_KEYS) {
            __syncthreads();  // the tile before has been used (and, the first time, the queries are in place)
            {
                const int key = tid >> 3, part = tid & 7;
                const int j = j0 + key;
                int page = -1;
                if (j >= kmin && j <= pb) page = table[pshift >= 0 ? (j >> pshift) : (j / page_size)];
                if (page >= 0) {
                    const int in_page = pshift >= 0 ? (j & (page_size - 1)) : (j % page_size);
                    const size_t row = ((size_t)page * nkv + hk) * page_size + in_page;
                    stage_row(k_cache + row * d, Ks + key * dp, d, part, 8, 1.0f);
                    stage_row(v_cache + row * (st.v_stride ? (size_t)st.v_stride : (size_t)dv), Vs + key * dvp, dv, part, 8, 1.0f);
                } else {
                    zero_row(Ks + key * dp, d, part, 8);
                    zero_row(Vs + key * dvp, dv, part, 8);
                }
            }
            __syncthreads();
            // 2 x 4 scores: rows r0, r0 + 1 against keys kx, kx + 8, kx + 16, kx + 24
            float sc[2][4];
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int c = 0; c < 4; ++c) sc[a][c] = 0.0f;
            const float* q0 = Qs + r0 * dp;
            const float* kb = Ks + kx * dp;
            for (int x = 0; x < d; x += 4) {
                const float4 qa = *reinterpret_cast<const float4*>(q0 + x);
                const float4 qb = *reinterpret_cast<const float4*>(q0 + dp + x);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float4 kv = *reinterpret_cast<const float4*>(kb + (size_t)(8 * c) * dp + x);
                    sc[0][c] = fmaf(qa.x, kv.x, fmaf(qa.y, kv.y, fmaf(qa.z, kv.z, fmaf(qa.w, kv.w, sc[0][c]))));
                    sc[1][c] = fmaf(qb.x, kv.x, fmaf(qb.y, kv.y, fmaf(qb.z, kv.z, fmaf(qb.w, kv.w, sc[1][c]))));
                }
            }
            // the rows' maxima and sums over the tile, among the eight lanes that share the rows
            float alpha[2];
#pragma unroll
            for (int a = 0; a < 2; ++a) {
                const int lo = first_key(rpos[a], window);
                float best = -INFINITY;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int j = j0 + kx + 8 * c;
                    const bool seen = rseq[a] == sq && j >= lo && j <= rpos[a];
                    sc[a][c] = seen ? with_terms(sc[a][c], rterm[a], j, rpos[a]) : -INFINITY;
                    best = fmaxf(best, sc[a][c]);
                }
#pragma unroll
                for (int o = 4; o > 0; o >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o));
                const float m_new = fmaxf(m[a], best);
                alpha[a] = (m_new == -INFINITY || m[a] == m_new) ? 1.0f : expf(m[a] - m_new);  // exp(-inf) = 0 at a row's first keys
                float sum = 0.0f;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float pw = sc[a][c] == -INFINITY ? 0.0f : expf(sc[a][c] - m_new);
                    Ps[(r0 + a) * (TL_KEYS + 1) + kx + 8 * c] = pw;
                    sum += pw;
                }
#pragma unroll
                for (int o = 4; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                l[a] = l[a] * alpha[a] + sum;
                m[a] = m_new;
            }
            __syncwarp();  // a row's weights are written and read by the same eight lanes
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int c = 0; c < NC; ++c)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[a][c][e] *= alpha[a];
            const float* p0 = Ps + r0 * (TL_KEYS + 1);
            for (int kj = 0; kj < TL_KEYS; ++kj) {
                const float pa0 = p0[kj], pa1 = p0[TL_KEYS + 1 + kj];
                const float* vrow = Vs + kj * dvp + kx * 4;
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    if (kx * 4 + 32 * c < dv) {
                        const float4 vv = *reinterpret_cast<const float4*>(vrow + 32 * c);
                        acc[0][c][0] = fmaf(pa0, vv.x, acc[0][c][0]), acc[0][c][1] = fmaf(pa0, vv.y, acc[0][c][1]);
                        acc[0][c][2] = fmaf(pa0, vv.z, acc[0][c][2]), acc[0][c][3] = fmaf(pa0, vv.w, acc[0][c][3]);
                        acc[1][c][0] = fmaf(pa1, vv.x, acc[1][c][0]), acc[1][c][1] = fmaf(pa1, vv.y, acc[1][c][1]);
                        acc[1][c][2] = fmaf(pa1, vv.z, acc[1][c][2]), acc[1][c][3] = fmaf(pa1, vv.w, acc[1][c][3]);
                    }
                }
            }
        }
        ta = tb + 1;
    }
#pragma unroll
    for (int a = 0; a < 2; ++a) {
        if (rt[a] >= t_end) continue;
        const float inv = 1.0f / (l[a] + sink_share(st, hk * g + (r0 + a) % g, m[a]));
        T* orow = out + (size_t)rt[a] * ldo + (size_t)(hk * g + (r0 + a) % g) * dv;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int col = kx * 4 + 32 * c;
            if (col < dv) {
#pragma unroll
                for (int e = 0; e < 4; ++e) orow[col + e] = from_float<T>(acc[a][c][e] * inv);
            }
        }
    }
}

size_t tiled_smem_bytes(int d, int dv) {
    return ((size_t)(TL_ROWS + TL_KEYS) * (d + 4) + (size_t)TL_KEYS * (dv + 4) + (size_t)TL_ROWS * (TL_KEYS + 1)) * sizeof(float);
}

bool tiled_takes(int dtype, int nh, int nkv, int d, int dv) {
    const int g = nkv > 0 ? nh / nkv : 0;
    const int unit = dtype == FERRIS_F32 ? 4 : 8;  // elements of a 16-byte piece
    return g >= 1 && g <= TL_ROWS && nh % nkv == 0 && d % unit == 0 && dv % unit == 0 && d <= 256 &&
           dv <= 256 && tiled_smem_bytes(d, dv) <= 200 * 1024;
}

template <typename T>
int launch_tiled(const void* q, int ldq, void* out, int ldo, const void* k_cache, const void* v_cache,
                 const int* block_tables, int max_blocks, const int* token_seq, const int* positions, int tokens, int nh,
                 int nkv, int d, int dv, int page_size, int window, float scale, const ScoreTerms st, cudaStream_t s) {
    const int qt = TL_ROWS / (nh / nkv);
    const dim3 grid((tokens + qt - 1) / qt, nkv), block(TL_THREADS);
    const size_t smem = tiled_smem_bytes(d, dv);
#define FERRIS_TL_LAUNCH(NC)                                                                                        \
    do {                                                                                                            \
        int e_ = ferris_allow_dynamic_smem((const void*)paged_attention_tiled_kernel<T, NC>, smem);                 \
        if (e_ != FERRIS_OK) return e_;                                                                             \
        ferris_launch(paged_attention_tiled_kernel<T, NC>, grid, block, smem, s, (const T*)q, ldq, (T*)out, ldo,   \
                      (const T*)k_cache, (const T*)v_cache, block_tables, max_blocks, token_seq, positions, tokens, \
                      nh, nkv, d, dv, page_size, window, scale, st);                                           \
    } while (0)
    if (dv <= 64)
        FERRIS_TL_LAUNCH(2);
    else if (dv <= 128)
        FERRIS_TL_LAUNCH(4);
    else
        FERRIS_TL_LAUNCH(8);
#undef FERRIS_TL_LAUNCH
    FERRIS_LAUNCH_CHECK();
}

}  // namespace

FERRIS_API int ferris_paged_attention_simt(const void* q, int ldq, void* out, int ldo, const void* k_cache,
                                           const void* v_cache, int dtype, const int* block_tables, int max_blocks,
                                           const int* token_seq, const int* positions, int tokens, int nh, int nkv,
                                           int d, int dv, int page_size, int window, float scale, const float* slopes,
                                           const float* log_r1, const float* log_r2, const float* sink, int v_stride,
                                           int kv_span, float* scratch, long long scratch_floats, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if ((log_r1 == nullptr) != (log_r2 == nullptr)) FERRIS_REFUSE("attention: the logarithmic penalty needs both of its numbers per head");
    if (slopes && log_r1) FERRIS_REFUSE("attention: a slope and a logarithmic penalty at once");
    if (v_stride < 0 || (v_stride > 0 && v_stride < dv)) FERRIS_REFUSE("attention: value rows %d apart hold no %d values", v_stride, dv);
    const ScoreTerms st = {slopes, log_r1, log_r2, sink, v_stride};
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0) FERRIS_REFUSE("attention: %d heads over %d kv heads", nh, nkv);
    if (d <= 0 || d > 32 * MAX_PER_LANE) FERRIS_REFUSE("attention: head size %d not in 1..%d", d, 32 * MAX_PER_LANE);
    if (dv <= 0 || dv > 32 * MAX_PER_LANE) FERRIS_REFUSE("attention: value head size %d not in 1..%d", dv, 32 * MAX_PER_LANE);
    if (page_size <= 0 || max_blocks <= 0) FERRIS_REFUSE("attention: page_size=%d max_blocks=%d", page_size, max_blocks);
    if (nh > 65535) FERRIS_REFUSE("attention: %d heads are more than one launch takes", nh);
    dim3 grid(tokens, nh);
    const size_t smem = (size_t)ATT_WARPS * (dv + 2) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype != FERRIS_F32 && dtype != FERRIS_BF16) FERRIS_REFUSE("attention: unknown dtype %d", dtype);
    // head sizes that eight lanes can share evenly, rows that start on 16 bytes: the kernel with eight lanes to a key
    const size_t elt = dtype == FERRIS_F32 ? 4 : 2;
    const bool aligned = (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0 && ((size_t)ldq * elt) % 16 == 0;
    // Query heads that share keys, where the caller brings scratch for shares of the keys (a step of single tokens):
    // the keys of a token are cut into as many shares as fill the SMs about three times over, of 64 keys at least.
    const int g = nh / nkv;
    if (scratch && kv_span > 0 && g % 2 == 0 && d % 16 == 0 && dv % 16 == 0 && d <= 256 && dv <= 256 && aligned) {
        const bool four = g % 4 == 0;
        const long long blocks = (long long)tokens * (nh / (four ? 4 : 2));
        static int sms = 0;
        if (sms <= 0) {
            int dev = 0;
            cudaGetDevice(&dev);
            if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        }
        // (with enough tokens and heads to fill the SMs four times over as they are, the kernel with a block per token
        // and head below is faster: a round of this one forms G x U scores per lane and is long.  1B-like sizes, a step
        // of 8 / 64 single tokens over 1,024 keys: 0.97 / 2.17 ms a step with shares, 1.13 / 1.92 ms without)
        long long splits = (long long)tokens * nh >= 4LL * sms ? 0 : (3LL * sms + blocks - 1) / blocks;
        const long long most = kv_span / 64 > 0 ? kv_span / 64 : 1;
        if (splits > most) splits = most;
        if (splits > 16) splits = 16;
        const long long fit = scratch_floats / ((long long)tokens * nh * (dv + 2));
        if (splits > fit) splits = fit;
        if (splits >= 1) {
            const int sp = (int)splits;
            if (dtype == FERRIS_F32) {
                if (four) launch_shared<float, 4>(q, ldq, out, ldo, k_cache, v_cache, block_tables, max_blocks, token_seq, positions, tokens, nh, nkv, d, dv, page_size, window, scale, st, sp, scratch, s);
                else launch_shared<float, 2>(q, ldq, out, ldo, k_cache, v_cache, block_tables, max_blocks, token_seq, positions, tokens, nh, nkv, d, dv, page_size, window, scale, st, sp, scratch, s);
            } else {
                if (four) launch_shared<bf16, 4>(q, ldq, out, ldo, k_cache, v_cache, block_tables, max_blocks, token_seq, positions, tokens, nh, nkv, d, dv, page_size, window, scale, st, sp, scratch, s);
                else launch_shared<bf16, 2>(q, ldq, out, ldo, k_cache, v_cache, block_tables, max_blocks, token_seq, positions, tokens, nh, nkv, d, dv, page_size, window, scale, st, sp, scratch, s);
            }
            FERRIS_LAUNCH_CHECK();
        }
    }
    if (d % 8 == 0 && dv % 8 == 0 && d <= 256 && dv <= 256 && aligned && (size_t)AL_GROUPS * (dv + 2) * sizeof(float) <= 48 * 1024) {
        if (dtype == FERRIS_F32)
            launch_lanes<float>(q, ldq, out, ldo, k_cache, v_cache, block_tables, max_blocks, token_seq, positions, tokens, nh, nkv, d, dv, page_size, window, scale, st, s);
        else
            launch_lanes<bf16>(q, ldq, out, ldo, k_cache, v_cache, block_tables, max_blocks, token_seq, positions, tokens, nh, nkv, d, dv, page_size, window, scale, st, s);
        FERRIS_LAUNCH_CHECK();
    }
    if (dtype == FERRIS_F32)
        ferris_launch(paged_attention_simt_kernel<float>, grid, dim3(ATT_THREADS), smem, s, (const float*)q, ldq, (float*)out, ldo, (const float*)k_cache, (const float*)v_cache, block_tables,
            max_blocks, token_seq, positions, nh, nkv, d, dv, page_size, window, scale, st);
    else if (dtype == FERRIS_BF16)
        ferris_launch(paged_attention_simt_kernel<bf16>, grid, dim3(ATT_THREADS), smem, s, (const bf16*)q, ldq, (bf16*)out, ldo, (const bf16*)k_cache, (const bf16*)v_cache, block_tables, max_blocks,
            token_seq, positions, nh, nkv, d, dv, page_size, window, scale, st);
    else
        FERRIS_REFUSE("attention: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}

// Whether ferris_paged_attention_tiled takes a geometry (head sizes in 16-byte pieces, at most 64 query heads to a
// kv head).
FERRIS_API int ferris_paged_attention_tiled_takes(int dtype, int nh, int nkv, int d, int dv) {
    return tiled_takes(dtype, nh, nkv, d, dv) ? 1 : 0;
}

// The same attention as ferris_paged_attention_simt (same arguments), for steps that bring portions of prompts.
FERRIS_API int ferris_paged_attention_tiled(const void* q, int ldq, void* out, int ldo, const void* k_cache,
                                            const void* v_cache, int dtype, const int* block_tables, int max_blocks,
                                            const int* token_seq, const int* positions, int tokens, int nh, int nkv,
                                            int d, int dv, int page_size, int window, float scale, const float* slopes,
                                            const float* log_r1, const float* log_r2, const float* sink, int v_stride,
                                            void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if ((log_r1 == nullptr) != (log_r2 == nullptr) || (slopes && log_r1)) FERRIS_REFUSE("tiled attention: one kind of distance penalty, with all its numbers");
    if (v_stride < 0 || (v_stride > 0 && v_stride < dv)) FERRIS_REFUSE("tiled attention: value rows %d apart hold no %d values", v_stride, dv);
    const ScoreTerms st = {slopes, log_r1, log_r2, sink, v_stride};
    if (dtype != FERRIS_F32 && dtype != FERRIS_BF16) FERRIS_REFUSE("attention: unknown dtype %d", dtype);
    if (page_size <= 0 || max_blocks <= 0) FERRIS_REFUSE("attention: page_size=%d max_blocks=%d", page_size, max_blocks);
    if (!tiled_takes(dtype, nh, nkv, d, dv)) FERRIS_REFUSE("tiled attention: %d heads over %d kv heads of %d / %d are not taken", nh, nkv, d, dv);
    const size_t elt = dtype == FERRIS_F32 ? 4 : 2;
    if ((((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) != 0 || ((size_t)ldq * elt) % 16 != 0)
        FERRIS_REFUSE("tiled attention: rows must start on 16 bytes");
    if (nkv > 65535) FERRIS_REFUSE("attention: %d kv heads are more than one launch takes", nkv);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        return launch_tiled<float>(q, ldq, out, ldo, k_cache, v_cache, block_tables, max_blocks, token_seq, positions, tokens, nh, nkv, d, dv, page_size, window, scale, st, s);
    return launch_tiled<bf16>(q, ldq, out, ldo, k_cache, v_cache, block_tables, max_blocks, token_seq, positions, tokens, nh, nkv, d, dv, page_size, window, scale, st, s);
}
