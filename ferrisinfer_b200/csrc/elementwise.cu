// Row-wise and element-wise kernels: token embedding gather, RMSNorm, SwiGLU, and the
// fused rotary-position + cache-write kernel.  All statistics, angles and products are fp32.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// Embedding gather: out[t, :] = table[ids[t], :], into the fp32 residual stream.
// Formula: crates/ferrisinfer-kernel/src/cpu/attention.rs:3-99 (a row copy; an id >= vocab is an error).
// An id outside [0, vocab) writes zeros and sets *status to 1 + the offending token index.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* ids,
                                    float* __restrict__ out, int hidden, int vocab, int* status) {
    FERRIS_TL_ENTRY();
    pdl_wait();
    pdl_launch_dependents();
    FERRIS_TL_BEGIN();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0 && status) atomicCAS(status, 0, t + 1);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.0f;
    } else {
        const T* row = table + (size_t)id * hidden;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_float(row[i]);
    }
    FERRIS_TL_END(1);
}

FERRIS_API int ferris_embed_gather(const void* table, int dtype, const int* ids, float* out, int tokens,
                                   int hidden, int vocab, int* status, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (hidden <= 0 || vocab <= 0) FERRIS_REFUSE("embed_gather: hidden=%d vocab=%d", hidden, vocab);
    const int threads = hidden >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        ferris_launch(embed_gather_kernel<float>, dim3(tokens), dim3(threads), 0, s, (const float*)table, ids, out, hidden, vocab, status);
    else if (dtype == FERRIS_BF16)
        ferris_launch(embed_gather_kernel<bf16>, dim3(tokens), dim3(threads), 0, s, (const bf16*)table, ids, out, hidden, vocab, status);
    else
        FERRIS_REFUSE("embed_gather: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// RMSNorm over rows of the fp32 residual stream:
//   ms = sum(x^2) / H;  r = 1 / sqrt(ms + eps);  y_j = (x_j * r) * w_j
// (crates/ferrisinfer-kernel/src/cpu/reduction.rs:35-41: eps inside the root, plain weight).
// With row_index, output row i is the norm of input row row_index[i] (used to norm only the
// rows whose logits are wanted).
// ---------------------------------------------------------------------------------------------
template <typename TOut>
__global__ void rmsnorm_kernel(const float* x, const float* __restrict__ w,
                               const int* __restrict__ row_index, TOut* __restrict__ out, int hidden,
                               float eps) {
    __shared__ float scratch[33];
    FERRIS_TL_ENTRY();
    pdl_wait();
    pdl_launch_dependents();
    FERRIS_TL_BEGIN();
    const int r = blockIdx.x;
    const int src = row_index ? row_index[r] : r;
    const float* xr = x + (size_t)src * hidden;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    TOut* o = out + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<TOut>((xr[i] * inv) * w[i]);
    FERRIS_TL_END(2);
}

__device__ __forceinline__ void store4(float* o, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(o) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(bf16* o, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(o) = v;
}

// The same norm, one WARP per row: the row (up to 4096 floats, a multiple of 4) is read once with 16-byte loads
// and stays in registers between the sum of squares and the scaling.  For long steps.
template <typename TOut, int VEC>  // VEC float4 per lane: hidden <= 128 * VEC
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float* x, const float* __restrict__ w,
                                                           const int* __restrict__ row_index, TOut* __restrict__ out,
                                                           int rows, int hidden, float eps) {
    FERRIS_TL_ENTRY();
    pdl_wait();
    pdl_launch_dependents();
    FERRIS_TL_BEGIN();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= rows) return;  // never the block's first thread, which ends the timeline record below
    const int src = row_index ? row_index[r] : r;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)src * hidden);
    const int n4 = hidden >> 2;
    float4 v[VEC];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
        const int i = lane + 32 * j;
        v[j] = i < n4 ? xr[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        ss = fmaf(v[j].x, v[j].x, ss);
        ss = fmaf(v[j].y, v[j].y, ss);
        ss = fmaf(v[j].z, v[j].z, ss);
        ss = fmaf(v[j].w, v[j].w, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    TOut* o = out + (size_t)r * hidden;
    const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
        const int i = lane + 32 * j;
        if (i < n4) {
            const float4 g = w4[i];
            store4(o + 4 * i, (v[j].x * inv) * g.x, (v[j].y * inv) * g.y, (v[j].z * inv) * g.z, (v[j].w * inv) * g.w);
        }
    }
    FERRIS_TL_END(6);
}

template <typename TOut>
static void launch_rmsnorm_rows(const float* x, const float* w, const int* row_index, TOut* out, int rows, int hidden,
                                float eps, cudaStream_t s) {
    const dim3 grid((rows + 7) / 8), block(256);
    if (hidden <= 1024)
        ferris_launch(rmsnorm_rows_kernel<TOut, 8>, grid, block, 0, s, x, w, row_index, out, rows, hidden, eps);
    else if (hidden <= 2048)
        ferris_launch(rmsnorm_rows_kernel<TOut, 16>, grid, block, 0, s, x, w, row_index, out, rows, hidden, eps);
    else
        ferris_launch(rmsnorm_rows_kernel<TOut, 32>, grid, block, 0, s, x, w, row_index, out, rows, hidden, eps);
}

FERRIS_API int ferris_rmsnorm(const float* x, const float* w, const int* row_index, void* out, int out_dtype,
                              int rows, int hidden, float eps, void* stream) {
    if (rows <= 0) return FERRIS_OK;
    if (hidden <= 0) FERRIS_REFUSE("rmsnorm: hidden=%d", hidden);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype != FERRIS_F32 && out_dtype != FERRIS_BF16) FERRIS_REFUSE("rmsnorm: unknown dtype %d", out_dtype);
    // A warp per row with the row in registers (16-byte loads, all of a row's in flight) wherever the row is aligned
    // and short enough; a block per row otherwise.  A warp per row also for few rows: the block's two barriers cost
    // more than seven more warps bring (decode step of 24 / 32 / 48 requests at the 0.5B sizes, two norm launches a
    // layer: 1.34 / 1.43 / 1.70 ms with a block per row below 64 rows, 1.28 / 1.37 / 1.65 ms with a warp per row).
    const bool aligned = ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)out & 15) == 0;
    if (hidden % 4 == 0 && hidden <= 4096 && aligned) {
        if (out_dtype == FERRIS_F32)
            launch_rmsnorm_rows<float>(x, w, row_index, (float*)out, rows, hidden, eps, s);
        else
            launch_rmsnorm_rows<bf16>(x, w, row_index, (bf16*)out, rows, hidden, eps, s);
        FERRIS_LAUNCH_CHECK();
    }
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    if (out_dtype == FERRIS_F32)
        ferris_launch(rmsnorm_kernel<float>, dim3(rows), dim3(threads), 0, s, x, w, row_index, (float*)out, hidden, eps);
    else
        ferris_launch(rmsnorm_kernel<bf16>, dim3(rows), dim3(threads), 0, s, x, w, row_index, (bf16*)out, hidden, eps);
    FERRIS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// SwiGLU: out[t, j] = silu(gate[t, j]) * up[t, j], silu(g) = g * 1 / (1 + exp(-g))
// (crates/ferrisinfer-kernel/src/cpu/elementwise.rs:189-190; crates/ferrisinfer-runtime/src/reference.rs:359-360).
// gate_up holds gate in columns [0, I) and up in [I, 2I) of each row.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* gate_up, T* __restrict__ out, int tokens, int inter) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t n = (size_t)tokens * inter;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / inter, j = i % inter;
        const float g = to_float(gate_up[t * 2 * inter + j]);
        const float u = to_float(gate_up[t * 2 * inter + inter + j]);
        const float sg = g * (1.0f / (1.0f + expf(-g)));
        out[i] = from_float<T>(u * sg);
    }
}

FERRIS_API int ferris_swiglu(const void* gate_up, void* out, int dtype, int tokens, int inter, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (inter <= 0) FERRIS_REFUSE("swiglu: intermediate=%d", inter);
    const size_t n = (size_t)tokens * inter;
    const int threads = 256;
    const int blocks = (int)((n + threads - 1) / threads < 148 * 16 ? (n + threads - 1) / threads : 148 * 16);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        ferris_launch(swiglu_kernel<float>, dim3(blocks), dim3(threads), 0, s, (const float*)gate_up, (float*)out, tokens, inter);
    else if (dtype == FERRIS_BF16)
        ferris_launch(swiglu_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, (const bf16*)gate_up, (bf16*)out, tokens, inter);
    else
        FERRIS_REFUSE("swiglu: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Rotary positions on q and k, and the write of k and v into the paged cache.
//   angle = float(pos) * inv_freq[i];  pairs (i, i + R/2), i < R/2 (rotate-half):
//   x_i' = x_i cos - x_{i+R/2} sin;  x_{i+R/2}' = x_{i+R/2} cos + x_i sin; dims >= R untouched
// (crates/ferrisinfer-kernel/src/cpu/attention.rs:1242-1292).  inv_freq is given by the host
// so that the engine and its plain reference agree on how the frequencies are formed.
//
// qkv: [T, (nh + 2 nkv) d] rows; q heads are rotated in place; k heads are rotated and stored
// to k_cache, v heads copied to v_cache, both laid out [page, kv head, slot in page, d].
// slot_mapping[t] = page * page_size + slot, or < 0 to write nothing for that token.
// With write_kv == 0 only q is rotated (a layer that reads another layer's cache).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_cache_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                        const float* __restrict__ inv_freq, const int* __restrict__ slot_mapping,
                                        T* __restrict__ k_cache, T* __restrict__ v_cache, int nh, int nkv, int d,
                                        int rotary, int page_size, int write_kv) {
    FERRIS_TL_ENTRY();
    pdl_wait();
    pdl_launch_dependents();
    FERRIS_TL_BEGIN();
    const int t = blockIdx.x;
    const int half = rotary / 2;
    const float pos = (float)positions[t];
    T* row = qkv + (size_t)t * (nh + 2 * nkv) * d;
    const int slot = write_kv ? slot_mapping[t] : -1;
    const int page = slot >= 0 ? slot / page_size : 0;
    const int in_page = slot >= 0 ? slot % page_size : 0;

    // rotate q and k heads: a thread takes a pair index and walks the heads, so that the sine and cosine of a
    // (token, pair) are formed once; with more threads than pairs, groups of threads share the heads
    const int rot_heads = nh + nkv;
    const int groups = half > 0 ? max(1, (int)blockDim.x / half) : 1;
    if (half > 0 && (int)threadIdx.x < groups * half) {
        const int i = threadIdx.x % half, g0 = threadIdx.x / half;
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        for (int h = g0; h < rot_heads; h += groups) {
            T* x = row + (size_t)h * d;
            const float lo = to_float(x[i]), hi = to_float(x[i + half]);
            const T nlo = from_float<T>(lo * cs - hi * sn);
            const T nhi = from_float<T>(hi * cs + lo * sn);
            if (h < nh) {
                x[i] = nlo;
                x[i + half] = nhi;
            } else if (slot >= 0) {
                T* kc = k_cache + (((size_t)page * nkv + (h - nh)) * page_size + in_page) * d;
                kc[i] = nlo;
                kc[i + half] = nhi;
            }
        }
    }
    if (slot < 0) {
        FERRIS_TL_END(3);
        return;
    }
    // unrotated tail of k, and all of v
    const int tail = d - rotary;
    for (int w = threadIdx.x; w < nkv * tail; w += blockDim.x) {
        const int h = w / tail, i = rotary + w % tail;
        k_cache[(((size_t)page * nkv + h) * page_size + in_page) * d + i] = row[(size_t)(nh + h) * d + i];
    }
    for (int w = threadIdx.x; w < nkv * d; w += blockDim.x) {
        const int h = w / d, i = w % d;
        v_cache[(((size_t)page * nkv + h) * page_size + in_page) * d + i] = row[(size_t)(nh + nkv + h) * d + i];
    }
    FERRIS_TL_END(3);
}

FERRIS_API int ferris_rope_cache_write(void* qkv, int dtype, const int* positions, const float* inv_freq,
                                       const int* slot_mapping, void* k_cache, void* v_cache, int tokens, int nh,
                                       int nkv, int d, int rotary, int page_size, int write_kv, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (nh <= 0 || nkv <= 0 || d <= 0 || page_size <= 0)
        FERRIS_REFUSE("rope_cache_write: nh=%d nkv=%d d=%d page_size=%d", nh, nkv, d, page_size);
    if (rotary < 0 || rotary > d || (rotary & 1)) FERRIS_REFUSE("rope_cache_write: rotary dims %d of %d", rotary, d);
    if (rotary > 0 && !inv_freq) FERRIS_REFUSE("rope_cache_write: no frequency table");
    if (write_kv && (!slot_mapping || !k_cache || !v_cache)) FERRIS_REFUSE("rope_cache_write: no cache to write");
    const int threads = 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        ferris_launch(rope_cache_write_kernel<float>, dim3(tokens), dim3(threads), 0, s, (float*)qkv, positions, inv_freq, slot_mapping,
                                                                  (float*)k_cache, (float*)v_cache, nh, nkv, d, rotary,
                                                                  page_size, write_kv);
    else if (dtype == FERRIS_BF16)
        ferris_launch(rope_cache_write_kernel<bf16>, dim3(tokens), dim3(threads), 0, s, (bf16*)qkv, positions, inv_freq, slot_mapping,
                                                                 (bf16*)k_cache, (bf16*)v_cache, nh, nkv, d, rotary,
                                                                 page_size, write_kv);
    else
        FERRIS_REFUSE("rope_cache_write: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// The rotation angles of a step, once for all layers that share the frequencies:
// out[t][i] = (cos, sin)(float(position[t]) * inv_freq[i]), the same fp32 expression as the kernel above.
// ---------------------------------------------------------------------------------------------
__global__ void rotary_angles_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                     float2* __restrict__ out, int tokens, int half) {
    FERRIS_TL_ENTRY();
    pdl_wait();
    pdl_launch_dependents();
    FERRIS_TL_BEGIN();
    const long long total = (long long)tokens * half;
    for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(w / half), i = (int)(w % half);
        float sn, cs;
        sincosf((float)positions[t] * inv_freq[i], &sn, &cs);
        out[w] = make_float2(cs, sn);
    }
    FERRIS_TL_END(9);
}

FERRIS_API int ferris_rotary_angles(const int* positions, const float* inv_freq, float* out, int tokens, int half,
                                    void* stream) {
    if (tokens <= 0 || half <= 0) return FERRIS_OK;
    const long long total = (long long)tokens * half;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 4096 ? (total + threads - 1) / threads : 4096);
    ferris_launch(rotary_angles_kernel, dim3(blocks), dim3(threads), 0, (cudaStream_t)stream, positions, inv_freq,
                  reinterpret_cast<float2*>(out), tokens, half);
    FERRIS_LAUNCH_CHECK();
}

FERRIS_TIMELINE_TU(elementwise)

// ---------------------------------------------------------------------------------------------
// Embedding with a scale and an additive sinusoidal position vector, into the fp32 residual stream:
//   out[t, 2i] = table[id, 2i] * scale + sin(float(pos_t) * f_i),  out[t, 2i+1] = table[id, 2i+1] * scale + cos(same)
// f (one frequency per pair of columns) comes from the host, which forms base^(-2i / hidden) in 64-bit and rounds
// once; the angle and its sine and cosine are fp32.  Ids outside [0, vocab) are reported as by embed_gather.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_sinusoid_kernel(const T* __restrict__ table, const int* ids, const int* positions,
                                      const float* __restrict__ freq, float scale, float* __restrict__ out, int hidden,
                                      int vocab, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int id = ids[t];
    const float pos = (float)positions[t];
    float* o = out + (size_t)t * hidden;
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0 && status) atomicCAS(status, 0, t + 1);
    const T* row = table + (size_t)(ok ? id : 0) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float pe = 0.0f;  // no frequencies: no position vector, the scaled table row alone
        if (freq) {
            const float angle = pos * freq[i >> 1];
            pe = (i & 1) ? cosf(angle) : sinf(angle);
        }
        o[i] = ok ? fmaf(to_float(row[i]), scale, pe) : 0.0f;
    }
}

FERRIS_API int ferris_embed_sinusoid(const void* table, int dtype, const int* ids, const int* positions,
                                     const float* freq, float scale, float* out, int tokens, int hidden, int vocab,
                                     int* status, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (hidden <= 0 || vocab <= 0) FERRIS_REFUSE("embed_sinusoid: hidden=%d vocab=%d", hidden, vocab);
    const int threads = hidden >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        ferris_launch(embed_sinusoid_kernel<float>, dim3(tokens), dim3(threads), 0, s, (const float*)table, ids, positions,
                      freq, scale, out, hidden, vocab, status);
    else if (dtype == FERRIS_BF16)
        ferris_launch(embed_sinusoid_kernel<bf16>, dim3(tokens), dim3(threads), 0, s, (const bf16*)table, ids, positions,
                      freq, scale, out, hidden, vocab, status);
    else
        FERRIS_REFUSE("embed_sinusoid: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// RMSNorm in groups: a row of `hidden` is cut into `groups` equal consecutive parts, each part is divided by its
// own sqrt(mean(part^2) + eps), and the whole is multiplied by w.  A warp per (row, group); statistics fp32.
// ---------------------------------------------------------------------------------------------
template <typename TOut>
__global__ void __launch_bounds__(256) grouped_rmsnorm_kernel(const float* x, const float* __restrict__ w,
                                                              const int* __restrict__ row_index, TOut* __restrict__ out,
                                                              int rows, int hidden, int groups, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (item >= (long long)rows * groups) return;
    const int r = (int)(item / groups), g = (int)(item % groups);
    const int n = hidden / groups;
    const int src = row_index ? row_index[r] : r;
    const float* xr = x + (size_t)src * hidden + (size_t)g * n;
    float ss = 0.0f;
    for (int i = lane; i < n; i += 32) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    TOut* o = out + (size_t)r * hidden + (size_t)g * n;
    const float* wg = w + (size_t)g * n;
    for (int i = lane; i < n; i += 32) o[i] = from_float<TOut>((xr[i] * inv) * wg[i]);
}

// Two such norms of the same rows with weights of their own (the two branches of a parallel block), in one launch.
template <typename TOut>
__global__ void __launch_bounds__(256) grouped_rmsnorm_pair_kernel(const float* x, const float* __restrict__ w1,
                                                                   const float* __restrict__ w2, TOut* __restrict__ out1,
                                                                   TOut* __restrict__ out2, int rows, int hidden,
                                                                   int groups, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (item >= (long long)rows * groups) return;
    const int r = (int)(item / groups), g = (int)(item % groups);
    const int n = hidden / groups;
    const size_t at = (size_t)r * hidden + (size_t)g * n;
    const float* xr = x + at;
    float ss = 0.0f;
    for (int i = lane; i < n; i += 32) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    const float* a = w1 + (size_t)g * n;
    const float* b = w2 + (size_t)g * n;
    for (int i = lane; i < n; i += 32) {
        const float v = xr[i] * inv;
        out1[at + i] = from_float<TOut>(v * a[i]);
        out2[at + i] = from_float<TOut>(v * b[i]);
    }
}

FERRIS_API int ferris_grouped_rmsnorm_pair(const float* x, const float* w1, const float* w2, void* out1, void* out2,
                                           int out_dtype, int rows, int hidden, int groups, float eps, void* stream) {
    if (rows <= 0) return FERRIS_OK;
    if (hidden <= 0 || groups <= 0 || hidden % groups) FERRIS_REFUSE("grouped rmsnorm: %d columns in %d groups", hidden, groups);
    const long long items = (long long)rows * groups;
    const dim3 grid((unsigned)((items + 7) / 8)), block(256);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == FERRIS_F32)
        ferris_launch(grouped_rmsnorm_pair_kernel<float>, grid, block, 0, s, x, w1, w2, (float*)out1, (float*)out2, rows, hidden, groups, eps);
    else if (out_dtype == FERRIS_BF16)
        ferris_launch(grouped_rmsnorm_pair_kernel<bf16>, grid, block, 0, s, x, w1, w2, (bf16*)out1, (bf16*)out2, rows, hidden, groups, eps);
    else
        FERRIS_REFUSE("grouped rmsnorm: unknown dtype %d", out_dtype);
    FERRIS_LAUNCH_CHECK();
}

FERRIS_API int ferris_grouped_rmsnorm(const float* x, const float* w, const int* row_index, void* out, int out_dtype,
                                      int rows, int hidden, int groups, float eps, void* stream) {
    if (rows <= 0) return FERRIS_OK;
    if (hidden <= 0 || groups <= 0 || hidden % groups) FERRIS_REFUSE("grouped rmsnorm: %d columns in %d groups", hidden, groups);
    const long long items = (long long)rows * groups;
    const dim3 grid((unsigned)((items + 7) / 8)), block(256);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == FERRIS_F32)
        ferris_launch(grouped_rmsnorm_kernel<float>, grid, block, 0, s, x, w, row_index, (float*)out, rows, hidden, groups, eps);
    else if (out_dtype == FERRIS_BF16)
        ferris_launch(grouped_rmsnorm_kernel<bf16>, grid, block, 0, s, x, w, row_index, (bf16*)out, rows, hidden, groups, eps);
    else
        FERRIS_REFUSE("grouped rmsnorm: unknown dtype %d", out_dtype);
    FERRIS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// h += x over n fp32 values (the embedding output that a repeated pass of a looped model takes in again).
// ---------------------------------------------------------------------------------------------
__global__ void add_f32_kernel(float* h, const float* x, long long n) {
    pdl_wait();
    pdl_launch_dependents();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        h[i] += x[i];
}

FERRIS_API int ferris_add_f32(float* h, const float* x, long long n, void* stream) {
    if (n <= 0) return FERRIS_OK;
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    ferris_launch(add_f32_kernel, dim3(blocks), dim3(threads), 0, (cudaStream_t)stream, h, x, n);
    FERRIS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Activations of a plain (ungated) feed-forward, out[i] = a(in[i]), fp32 arithmetic.
//   kind 0, xIELU with two learned numbers (p, q) in `params`:
//     z > 0:  softplus(p) z^2 + z / 2;   z <= 0:  (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2
//   kind 1, SiLU: z / (1 + exp(-z)).   kind 2: the square of max(z, 0).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

template <typename T>
__global__ void activation_kernel(const T* in, T* out, long long n, int kind,
                                  const float* __restrict__ params) {
    pdl_wait();
    pdl_launch_dependents();
    float a = 0.0f, b = 0.0f;
    if (kind == 0) {
        a = softplus_f(params[0]);
        b = 0.5f + softplus_f(params[1]);
    }
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float z = to_float(in[i]);
        float r;
        if (kind == 0)
            r = z > 0.0f ? fmaf(a * z, z, 0.5f * z) : fmaf(b, expm1f(z) - z, 0.5f * z);
        else if (kind == 2)
            r = z > 0.0f ? z * z : 0.0f;
        else
            r = z / (1.0f + expf(-z));
        out[i] = from_float<T>(r);
    }
}

// The same, sixteen bytes a thread at a time (eight bf16 values or four floats), where the count and the addresses allow.
__device__ __forceinline__ float activation_value(float z, int kind, float a, float b) {
    if (kind == 0) return z > 0.0f ? fmaf(a * z, z, 0.5f * z) : fmaf(b, expm1f(z) - z, 0.5f * z);
    if (kind == 2) return z > 0.0f ? z * z : 0.0f;
    return z / (1.0f + expf(-z));
}

template <typename T>
__global__ void activation_vec_kernel(const uint4* in, uint4* out, long long n16, int kind, const float* __restrict__ params) {
    pdl_wait();
    pdl_launch_dependents();
    float a = 0.0f, b = 0.0f;
    if (kind == 0) {
        a = softplus_f(params[0]);
        b = 0.5f + softplus_f(params[1]);
    }
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x) {
        uint4 u = in[i];
        uint32_t* w = reinterpret_cast<uint32_t*>(&u);
        if (sizeof(T) == 4) {
#pragma unroll
            for (int k = 0; k < 4; ++k) w[k] = __float_as_uint(activation_value(__uint_as_float(w[k]), kind, a, b));
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float lo = activation_value(__uint_as_float(w[k] << 16), kind, a, b);
                const float hi = activation_value(__uint_as_float(w[k] & 0xffff0000u), kind, a, b);
                const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
                w[k] = *reinterpret_cast<const uint32_t*>(&pair);
            }
        }
        out[i] = u;
    }
}

FERRIS_API int ferris_activation(const void* in, void* out, int dtype, long long n, int kind, const float* params,
                                 void* stream) {
    if (n <= 0) return FERRIS_OK;
    if (kind < 0 || kind > 2) FERRIS_REFUSE("activation: unknown kind %d", kind);
    if (kind == 0 && !params) FERRIS_REFUSE("activation: xIELU needs its two numbers");
    if (dtype != FERRIS_F32 && dtype != FERRIS_BF16) FERRIS_REFUSE("activation: unknown dtype %d", dtype);
    const int threads = 256;
    cudaStream_t s = (cudaStream_t)stream;
    const long long per16 = dtype == FERRIS_F32 ? 4 : 8;
    if (n % per16 == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
        const long long n16 = n / per16, want = (n16 + threads - 1) / threads;
        const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
        if (dtype == FERRIS_F32)
            ferris_launch(activation_vec_kernel<float>, dim3(blocks), dim3(threads), 0, s, (const uint4*)in, (uint4*)out, n16, kind, params);
        else
            ferris_launch(activation_vec_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, (const uint4*)in, (uint4*)out, n16, kind, params);
        FERRIS_LAUNCH_CHECK();
    }
    const long long want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (dtype == FERRIS_F32)
        ferris_launch(activation_kernel<float>, dim3(blocks), dim3(threads), 0, s, (const float*)in, (float*)out, n, kind, params);
    else
        ferris_launch(activation_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, (const bf16*)in, (bf16*)out, n, kind, params);
    FERRIS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// What stands between the q/k/v product and attention where positions do not rotate anything:
//   q and k heads divided by their own sqrt(mean(.^2) + eps) when `unit_norm` (an RMS norm without a weight);
//   q multiplied by a temperature that grows with the position, 1 + coef * ln(floor((pos + 1) / every) + 1),
//   when every > 0; k and v stored into the paged cache (k heads of d, v heads of dv).
// qkv rows: [nh d | nkv d | nkv dv]; q is rewritten in place.  One block per token, a warp per head in turn.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) qk_prepare_cache_write_kernel(
    T* __restrict__ qkv, int ld, const int* __restrict__ positions, const int* __restrict__ slot_mapping,
    T* __restrict__ k_cache, T* __restrict__ v_cache, int nh, int nkv, int d, int dv, int page_size, int unit_norm,
    float eps, float temp_coef, int temp_every, int write_kv) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int pos = positions[t];
    T* row = qkv + (size_t)t * ld;
    const int slot = write_kv ? slot_mapping[t] : -1;
    const int page = slot >= 0 ? slot / page_size : 0;
    const int in_page = slot >= 0 ? slot % page_size : 0;
    const float temp = temp_every > 0 ? 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f) : 1.0f;
    for (int h = warp; h < nh + nkv; h += warps) {
        T* x = row + (size_t)h * d;
        float ss = 0.0f;
        if (unit_norm) {
            for (int i = lane; i < d; i += 32) {
                const float v = to_float(x[i]);
                ss = fmaf(v, v, ss);
            }
            ss = warp_sum(ss);
        }
        float f = unit_norm ? 1.0f / sqrtf(ss / (float)d + eps) : 1.0f;
        if (h < nh) {
            f *= temp;
            for (int i = lane; i < d; i += 32) x[i] = from_float<T>(to_float(x[i]) * f);
        } else if (slot >= 0) {
            T* kc = k_cache + (((size_t)page * nkv + (h - nh)) * page_size + in_page) * d;
            for (int i = lane; i < d; i += 32) kc[i] = from_float<T>(to_float(x[i]) * f);
        }
    }
    if (slot < 0) return;
    const T* vrow = row + (size_t)(nh + nkv) * d;
    for (int w = threadIdx.x; w < nkv * dv; w += blockDim.x) {
        const int h = w / dv, i = w % dv;
        v_cache[(((size_t)page * nkv + h) * page_size + in_page) * dv + i] = vrow[w];
    }
}

FERRIS_API int ferris_qk_prepare_cache_write(void* qkv, int ld, int dtype, const int* positions, const int* slot_mapping,
                                             void* k_cache, void* v_cache, int tokens, int nh, int nkv, int d, int dv,
                                             int page_size, int unit_norm, float eps, float temp_coef, int temp_every,
                                             int write_kv, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (nh <= 0 || nkv <= 0 || d <= 0 || dv <= 0 || page_size <= 0)
        FERRIS_REFUSE("qk_prepare: nh=%d nkv=%d d=%d dv=%d page_size=%d", nh, nkv, d, dv, page_size);
    if (ld < (nh + nkv) * d + nkv * dv) FERRIS_REFUSE("qk_prepare: rows of %d are too short", ld);
    if (write_kv && (!slot_mapping || !k_cache || !v_cache)) FERRIS_REFUSE("qk_prepare: no cache to write");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        ferris_launch(qk_prepare_cache_write_kernel<float>, dim3(tokens), dim3(128), 0, s, (float*)qkv, ld, positions,
                      slot_mapping, (float*)k_cache, (float*)v_cache, nh, nkv, d, dv, page_size, unit_norm, eps, temp_coef,
                      temp_every, write_kv);
    else if (dtype == FERRIS_BF16)
        ferris_launch(qk_prepare_cache_write_kernel<bf16>, dim3(tokens), dim3(128), 0, s, (bf16*)qkv, ld, positions,
                      slot_mapping, (bf16*)k_cache, (bf16*)v_cache, nh, nkv, d, dv, page_size, unit_norm, eps, temp_coef,
                      temp_every, write_kv);
    else
        FERRIS_REFUSE("qk_prepare: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Dynamic tanh, a norm without statistics: out[r, i] = tanh(alpha * x[src(r), i]) * w[i] + b[i], alpha one learned
// number (read from the device).  fp32 arithmetic, tanhf in full precision; the output in the activations' type.
// Rows of a multiple of four elements go 16 bytes a thread.
// ---------------------------------------------------------------------------------------------
template <typename TOut>
__global__ void __launch_bounds__(256) dynamic_tanh_kernel(const float* x, const float* __restrict__ w,
                                                           const float* __restrict__ b, const float* __restrict__ alpha,
                                                           const int* __restrict__ row_index, TOut* __restrict__ out,
                                                           int rows, int hidden) {
    const float a = alpha[0];
    pdl_wait();
    pdl_launch_dependents();
    const size_t n = (size_t)rows * hidden;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t r = e / hidden;
        const int i = (int)(e % hidden);
        const size_t src = row_index ? (size_t)row_index[r] : r;
        out[e] = from_float<TOut>(fmaf(tanhf(a * x[src * hidden + i]), w[i], b[i]));
    }
}

template <typename TOut>
__global__ void __launch_bounds__(256) dynamic_tanh_vec_kernel(const float* x, const float* __restrict__ w,
                                                               const float* __restrict__ b,
                                                               const float* __restrict__ alpha,
                                                               const int* __restrict__ row_index, TOut* __restrict__ out,
                                                               int rows, int hidden) {
    const float a = alpha[0];
    pdl_wait();
    pdl_launch_dependents();
    const int n4 = hidden >> 2;
    const size_t n = (size_t)rows * n4;
    const float4* w4 = reinterpret_cast<const float4*>(w);
    const float4* b4 = reinterpret_cast<const float4*>(b);
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t r = e / n4;
        const int i = (int)(e % n4);
        const size_t src = row_index ? (size_t)row_index[r] : r;
        const float4 v = reinterpret_cast<const float4*>(x + src * hidden)[i];
        const float4 g = w4[i], c = b4[i];
        store4(out + r * hidden + 4 * i, fmaf(tanhf(a * v.x), g.x, c.x), fmaf(tanhf(a * v.y), g.y, c.y),
               fmaf(tanhf(a * v.z), g.z, c.z), fmaf(tanhf(a * v.w), g.w, c.w));
    }
}

FERRIS_API int ferris_dynamic_tanh(const float* x, const float* w, const float* b, const float* alpha,
                                   const int* row_index, void* out, int out_dtype, int rows, int hidden, void* stream) {
    if (rows <= 0) return FERRIS_OK;
    if (hidden <= 0 || !w || !b || !alpha) FERRIS_REFUSE("dynamic tanh: hidden=%d, or a tensor is missing", hidden);
    if (out_dtype != FERRIS_F32 && out_dtype != FERRIS_BF16) FERRIS_REFUSE("dynamic tanh: unknown dtype %d", out_dtype);
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = hidden % 4 == 0 && (((uintptr_t)x | (uintptr_t)w | (uintptr_t)b | (uintptr_t)out) & 15) == 0;
    const size_t n = (size_t)rows * (vec ? hidden / 4 : hidden);
    const size_t want = (n + 255) / 256;
    const dim3 grid((unsigned)(want < 148 * 16 ? want : 148 * 16)), block(256);
    if (vec) {
        if (out_dtype == FERRIS_F32)
            ferris_launch(dynamic_tanh_vec_kernel<float>, grid, block, 0, s, x, w, b, alpha, row_index, (float*)out, rows, hidden);
        else
            ferris_launch(dynamic_tanh_vec_kernel<bf16>, grid, block, 0, s, x, w, b, alpha, row_index, (bf16*)out, rows, hidden);
    } else {
        if (out_dtype == FERRIS_F32)
            ferris_launch(dynamic_tanh_kernel<float>, grid, block, 0, s, x, w, b, alpha, row_index, (float*)out, rows, hidden);
        else
            ferris_launch(dynamic_tanh_kernel<bf16>, grid, block, 0, s, x, w, b, alpha, row_index, (bf16*)out, rows, hidden);
    }
    FERRIS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Soft cap of logits, in place: z <- cap * tanh(z / cap).  fp32.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) softcap_kernel(float* z, long long n, float cap) {
    pdl_wait();
    pdl_launch_dependents();
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x)
        z[e] = cap * tanhf(z[e] / cap);
}

FERRIS_API int ferris_softcap(float* z, long long n, float cap, void* stream) {
    if (n <= 0) return FERRIS_OK;
    if (!(cap > 0.0f)) FERRIS_REFUSE("softcap: the cap must be positive, found %g", (double)cap);
    const long long want = (n + 255) / 256;
    ferris_launch(softcap_kernel, dim3((unsigned)(want < 148 * 16 ? want : 148 * 16)), dim3(256), 0, (cudaStream_t)stream,
                  z, n, cap);
    FERRIS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// The gated feed-forward's activation as a kernel of its own: out[t, j] = f(gate_up[t, j], gate_up[t, I + j]) with f one
// of the kinds of ferris_gated_act; rows of gate_up ld apart.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void gated_activation_kernel(const T* gate_up, int ld, T* __restrict__ out, int tokens, int inter, int kind,
                                        float limit) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t n = (size_t)tokens * inter;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / inter, j = i % inter;
        const float g = to_float(gate_up[t * ld + j]);
        const float u = to_float(gate_up[t * ld + inter + j]);
        out[i] = from_float<T>(ferris_gated_act(g, u, kind, limit));
    }
}

FERRIS_API int ferris_gated_activation(const void* gate_up, int ld, void* out, int dtype, int tokens, int inter, int kind,
                                       float limit, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (inter <= 0 || ld < 2 * inter) FERRIS_REFUSE("gated activation: intermediate=%d in rows of %d", inter, ld);
    if (kind < 0 || kind > 2) FERRIS_REFUSE("gated activation: unknown kind %d", kind);
    const size_t n = (size_t)tokens * inter;
    const int threads = 256;
    const int blocks = (int)((n + threads - 1) / threads < 148 * 16 ? (n + threads - 1) / threads : 148 * 16);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        ferris_launch(gated_activation_kernel<float>, dim3(blocks), dim3(threads), 0, s, (const float*)gate_up, ld, (float*)out, tokens, inter, kind, limit);
    else if (dtype == FERRIS_BF16)
        ferris_launch(gated_activation_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, (const bf16*)gate_up, ld, (bf16*)out, tokens, inter, kind, limit);
    else
        FERRIS_REFUSE("gated activation: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// out[t, j] = x[t, j] * a(gate[t, j]) * scale, a = sigmoid (kind 0) or SiLU (kind 1); rows ldx / ldg / ldo apart; out may
// be x.  The gate of an attention's output: the heads side by side times a function of a projection of the layer's input.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void gate_mul_kernel(const T* x, int ldx, const T* gate, int ldg, T* out, int ldo, int rows, int n, int kind,
                                float scale) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t total = (size_t)rows * n;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / n, j = i % n;
        const float z = to_float(gate[t * ldg + j]);
        const float sg = 1.0f / (1.0f + expf(-z));
        out[t * ldo + j] = from_float<T>(to_float(x[t * ldx + j]) * (kind == 1 ? z * sg : sg) * scale);
    }
}

FERRIS_API int ferris_gate_mul(const void* x, int ldx, const void* gate, int ldg, void* out, int ldo, int dtype, int rows,
                               int n, int kind, float scale, void* stream) {
    if (rows <= 0) return FERRIS_OK;
    if (n <= 0 || ldx < n || ldg < n || ldo < n) FERRIS_REFUSE("gate: %d columns in rows of %d, %d, %d", n, ldx, ldg, ldo);
    if (kind != 0 && kind != 1) FERRIS_REFUSE("gate: unknown kind %d", kind);
    const size_t total = (size_t)rows * n;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        ferris_launch(gate_mul_kernel<float>, dim3(blocks), dim3(threads), 0, s, (const float*)x, ldx, (const float*)gate, ldg, (float*)out, ldo, rows, n, kind, scale);
    else if (dtype == FERRIS_BF16)
        ferris_launch(gate_mul_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, (const bf16*)x, ldx, (const bf16*)gate, ldg, (bf16*)out, ldo, rows, n, kind, scale);
    else
        FERRIS_REFUSE("gate: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}

// logits <- logits * scale in place; fp32.
__global__ void scale_kernel(float* x, long long n, float scale) {
    pdl_wait();
    pdl_launch_dependents();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) x[i] *= scale;
}

FERRIS_API int ferris_scale(float* x, long long n, float scale, void* stream) {
    if (n <= 0) return FERRIS_OK;
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    ferris_launch(scale_kernel, dim3((unsigned)(want < 148 * 16 ? want : 148 * 16)), dim3(threads), 0, (cudaStream_t)stream, x, n, scale);
    FERRIS_LAUNCH_CHECK();
}
