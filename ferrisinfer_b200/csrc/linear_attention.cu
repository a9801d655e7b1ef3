// Linear attention with a fixed decay per head (a recurrence over a state of fixed size instead of a softmax over
// cached keys), and the gated norm that follows it.
//
//   S_t = decay_h * S_(t-1) + k_t v_t^T        S: [dim, vdim] per (request, head), fp32, zero at admission
//   o_t = S_t^T q_t                            no other scale
//
// The columns of S do not depend on one another, so a warp owns eight of them for one (request, head) and walks
// the request's tokens of the step in order: a lane holds rows lane, lane + 32, ... of its eight columns in
// registers, updates them with fp32 FMAs, and the eight dot products with q are summed over the warp.  The four
// warps of a block share a head: they bring q, k and their 32 columns of v of eight tokens at a time into shared
// memory, activation applied once, and then each walks those tokens alone.  A step of single tokens and a portion
// of a prompt are the same loop, and a long portion is cut into segments that run side by side (see the kernel).  The state lies
// transposed in memory, [slot, head, vdim, dim], so that a warp reads and writes whole rows of it.
// q, k, v may be passed through SiLU on the way in (`silu`), in fp32 whatever the storage type; q and k may be
// rotated by their positions there, and k scaled (RotaryArgs): what enters the recurrence is then fp32 throughout.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int LA_COLS = 8;
constexpr int LA_WARPS = 4;
constexpr int LA_STAGE = 8;      // tokens whose q, k, v stand in shared memory at a time
constexpr int LA_MAX_DIM = 256;  // largest head size

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// Rotary positions on q and k on their way in (positions null: none), and a factor on k after them.  The first
// `rotary` elements of a head are rotated by the token's position: the pair (u, v), elements (i, i + rotary / 2)
// or, `interleaved`, (2i, 2i + 1), becomes (u c - v s, v c + u s) with c = mag cos(pos * freq[i]), s = mag sin(same);
// position x frequency is one fp32 product, sine and cosine are in full precision.
struct RotaryArgs {
    const int* positions;
    const float* freq;
    int rotary, interleaved;
    float mag, k_scale;
};

// Eight sums over the warp's lanes with nine shuffles instead of forty: at each of the first three steps a lane
// hands half of its partial sums to its partner and keeps the other half.  Every lane returns the sum of column
// ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1); the order of the additions is fixed.
__device__ __forceinline__ float reduce_columns(const float (&o)[LA_COLS], int lane) {
    const unsigned full = 0xffffffffu;
    const bool h1 = lane & 16, h2 = lane & 8, h3 = lane & 4;
    float a[4], b[2];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const float send = h1 ? o[c] : o[c + 4], keep = h1 ? o[c + 4] : o[c];
        a[c] = keep + __shfl_xor_sync(full, send, 16);
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const float send = h2 ? a[c] : a[c + 2], keep = h2 ? a[c + 2] : a[c];
        b[c] = keep + __shfl_xor_sync(full, send, 8);
    }
    const float send = h3 ? b[0] : b[1], keep = h3 ? b[1] : b[0];
    float r = keep + __shfl_xor_sync(full, send, 4);
    r += __shfl_xor_sync(full, r, 2);
    r += __shfl_xor_sync(full, r, 1);
    return r;
}

// Long portions of prompts are cut into segments of `seg_len` tokens that run side by side (the recurrence is linear
// in the state): MODE 1 sums each segment's own k v^T from a zero state into `scratch`; the combine kernel below turns
// those into the state at each segment's start; MODE 2 then runs each segment from that state and writes the outputs,
// the last segment of a request also the request's state.  MODE 0 is the whole request in one go, from and to its slot
// (single tokens and short portions).  A segment's place in `scratch` is (its first row / seg_len) + its request's
// index in the step, which no two segments share.
template <typename T, int RPL, int MODE>  // RPL rows of the state per lane: dim <= 32 * RPL
__global__ void __launch_bounds__(LA_WARPS * 32) linear_attention_scan_kernel(
    const T* qkv, int ld, int q_off, int k_off, int v_off, float* __restrict__ out, int ldo, float* state,
    float* scratch, const float* __restrict__ decay, const int* __restrict__ seq_q_start,
    const int* __restrict__ seq_state_slot, int heads, int dim, int vdim, int silu, int write_state, int seg_len,
    int segs_max, const RotaryArgs rot) {
    pdl_wait();
    pdl_launch_dependents();
    // q, k and this block's 32 columns of v of LA_STAGE tokens at a time, activation applied once, for all four warps
    __shared__ float stage[LA_STAGE][2 * LA_MAX_DIM + LA_COLS * LA_WARPS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y;
    const int seq = MODE == 0 ? blockIdx.x : blockIdx.x / segs_max;
    const int seg = MODE == 0 ? 0 : blockIdx.x % segs_max;
    const int bcol0 = blockIdx.z * LA_WARPS * LA_COLS;  // the block's first column
    const int col0 = bcol0 + warp * LA_COLS;
    const bool mine_cols = col0 < vdim;  // a warp beyond the last column only helps to stage
    int row0 = seq_q_start[seq];
    int row1 = seq_q_start[seq + 1];
    bool last = true;
    if (MODE != 0) {
        row0 += seg * seg_len;
        if (row0 >= row1) return;  // the whole block
        last = row0 + seg_len >= row1;
        if (!last) row1 = row0 + seg_len;
        if (MODE == 1 && last) return;  // nobody starts from the end of the last segment
    }
    if (row1 <= row0) return;
    const float lam = decay[h];
    const size_t tile = ((size_t)h * vdim + (mine_cols ? col0 : 0)) * dim;
    const size_t per_state = (size_t)heads * vdim * dim;
    float* slot_state = state + (size_t)seq_state_slot[seq] * per_state + tile;
    float* seg_state = MODE == 0 ? slot_state : scratch + (size_t)(row0 / seg_len + seq) * per_state + tile;
    float S[LA_COLS][RPL];
#pragma unroll
    for (int c = 0; c < LA_COLS; ++c)
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
            const int i = lane + 32 * r;
            S[c][r] = (MODE != 1 && mine_cols && col0 + c < vdim && i < dim) ? seg_state[(size_t)c * dim + i] : 0.0f;
        }
    const int my_col = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
    const int bcols = min(LA_COLS * LA_WARPS, vdim - bcol0);
    for (int t0 = row0; t0 < row1; t0 += LA_STAGE) {
        const int nt = min(LA_STAGE, row1 - t0);
        __syncthreads();  // the tokens staged before have been used
        for (int tt = warp; tt < nt; tt += LA_WARPS) {  // a warp per token
            const T* row = qkv + (size_t)(t0 + tt) * ld;
            for (int e = lane; e < dim; e += 32) {
                const float a = to_float(row[k_off + h * dim + e]);
                stage[tt][e] = silu ? silu_f(a) : a;
            }
            if (MODE != 1) {  // no queries in the pass that only sums
                for (int e = lane; e < dim; e += 32) {
                    const float a = to_float(row[q_off + h * dim + e]);
                    stage[tt][LA_MAX_DIM + e] = silu ? silu_f(a) : a;
                }
            }
            for (int e = lane; e < bcols; e += 32) {
                const float a = to_float(row[v_off + h * vdim + bcol0 + e]);
                stage[tt][2 * LA_MAX_DIM + e] = silu ? silu_f(a) : a;
            }
            if (rot.positions || rot.k_scale != 1.0f) {
                __syncwarp();
                const int rotary = rot.positions ? rot.rotary : 0, half = rotary >> 1;
                const float p = rot.positions ? (float)rot.positions[t0 + tt] : 0.0f;
                for (int f = lane; f < half; f += 32) {
                    float sn, cs;
                    sincosf(p * rot.freq[f], &sn, &cs);
                    sn *= rot.mag, cs *= rot.mag;
                    const int iu = rot.interleaved ? 2 * f : f, iv = rot.interleaved ? 2 * f + 1 : f + half;
                    const float ku = stage[tt][iu], kv = stage[tt][iv];
                    stage[tt][iu] = (ku * cs - kv * sn) * rot.k_scale;
                    stage[tt][iv] = (kv * cs + ku * sn) * rot.k_scale;
                    if (MODE != 1) {
                        const float qu = stage[tt][LA_MAX_DIM + iu], qv = stage[tt][LA_MAX_DIM + iv];
                        stage[tt][LA_MAX_DIM + iu] = qu * cs - qv * sn;
                        stage[tt][LA_MAX_DIM + iv] = qv * cs + qu * sn;
                    }
                }
                for (int e = rotary + lane; e < dim; e += 32) stage[tt][e] *= rot.k_scale;
            }
        }
        __syncthreads();
        if (!mine_cols) continue;
        for (int tt = 0; tt < nt; ++tt) {
            float kk[RPL], qq[RPL], vv[LA_COLS];
#pragma unroll
            for (int r = 0; r < RPL; ++r) {
                const int i = lane + 32 * r;
                kk[r] = i < dim ? stage[tt][i] : 0.0f;
                qq[r] = (MODE != 1 && i < dim) ? stage[tt][LA_MAX_DIM + i] : 0.0f;
            }
#pragma unroll
            for (int c = 0; c < LA_COLS; ++c) vv[c] = col0 + c < vdim ? stage[tt][2 * LA_MAX_DIM + warp * LA_COLS + c] : 0.0f;
            float o[LA_COLS];
#pragma unroll
            for (int c = 0; c < LA_COLS; ++c) {
                float acc = 0.0f;
#pragma unroll
                for (int r = 0; r < RPL; ++r) {
                    S[c][r] = fmaf(kk[r], vv[c], lam * S[c][r]);
                    if (MODE != 1) acc = fmaf(S[c][r], qq[r], acc);
                }
                o[c] = acc;
            }
            if (MODE != 1) {
                const float sum = reduce_columns(o, lane);
                if ((lane & 3) == 0 && col0 + my_col < vdim) out[(size_t)(t0 + tt) * ldo + h * vdim + col0 + my_col] = sum;
            }
        }
    }
    float* dst = MODE == 1 ? seg_state : slot_state;
    if (mine_cols && (MODE == 1 || (write_state && last))) {
#pragma unroll
        for (int c = 0; c < LA_COLS; ++c)
#pragma unroll
            for (int r = 0; r < RPL; ++r) {
                const int i = lane + 32 * r;
                if (col0 + c < vdim && i < dim) dst[(size_t)c * dim + i] = S[c][r];
            }
    }
}

// Between the two passes over segments: scratch holds each full segment's own sum; afterwards it holds the state at
// each segment's start, S_start(0) = the request's state, S_start(s + 1) = decay^seg_len S_start(s) + sum(s).
__global__ void __launch_bounds__(256) linear_attention_combine_kernel(
    const float* state, float* scratch, const float* __restrict__ decay, const int* __restrict__ seq_q_start,
    const int* __restrict__ seq_state_slot, int heads, int dim, int vdim, int seg_len) {
    pdl_wait();
    pdl_launch_dependents();
    const int seq = blockIdx.y;
    const size_t per_state = (size_t)heads * vdim * dim;
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= per_state) return;
    const int row0 = seq_q_start[seq], row1 = seq_q_start[seq + 1];
    if (row1 <= row0) return;
    const int h = (int)(e / ((size_t)vdim * dim));
    const float lam = decay[h];
    float step = 1.0f;
    for (int i = 0; i < seg_len; ++i) step *= lam;  // the factor a state takes over one full segment
    float S = state[(size_t)seq_state_slot[seq] * per_state + e];
    for (int r = row0; r < row1; r += seg_len) {
        float* at = scratch + (size_t)(r / seg_len + seq) * per_state + e;
        const bool full = r + seg_len < row1;
        const float own = full ? *at : 0.0f;
        *at = S;
        S = fmaf(step, S, own);
    }
}

// out[t, i] = (o[t, i] / sqrt(mean_i(o[t, :]^2) + eps)) * w[i] * sigmoid(g[t, i]); o fp32, g and out in the
// activations' type.  A block per row.
template <typename T>
__global__ void __launch_bounds__(256) gated_rmsnorm_kernel(const float* o, int ldi, const T* g, int ldg,
                                                            const float* __restrict__ w, T* __restrict__ out, int ldo,
                                                            int n, float eps) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const float* orow = o + (size_t)t * ldi;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = orow[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    const T* grow = g + (size_t)t * ldg;
    T* dst = out + (size_t)t * ldo;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float gate = 1.0f / (1.0f + expf(-to_float(grow[i])));
        dst[i] = from_float<T>(((orow[i] * inv) * w[i]) * gate);
    }
}

template <typename T, int MODE>
void launch_scan_mode(const void* qkv, int ld, int q_off, int k_off, int v_off, float* out, int ldo, float* state,
                      float* scratch, const float* decay, const int* seq_q_start, const int* seq_state_slot, int seqs,
                      int heads, int dim, int vdim, int silu, int write_state, int seg_len, int segs_max, const RotaryArgs rot,
                      cudaStream_t s) {
    const dim3 grid(MODE == 0 ? seqs : seqs * segs_max, heads, (vdim + LA_COLS * LA_WARPS - 1) / (LA_COLS * LA_WARPS));
    const dim3 block(LA_WARPS * 32);
#define FERRIS_LA_LAUNCH(RPL)                                                                                       \
    ferris_launch(linear_attention_scan_kernel<T, RPL, MODE>, grid, block, 0, s, (const T*)qkv, ld, q_off, k_off,   \
                  v_off, out, ldo, state, scratch, decay, seq_q_start, seq_state_slot, heads, dim, vdim, silu,       \
                  write_state, seg_len, segs_max, rot)
    if (dim <= 32)
        FERRIS_LA_LAUNCH(1);
    else if (dim <= 64)
        FERRIS_LA_LAUNCH(2);
    else if (dim <= 128)
        FERRIS_LA_LAUNCH(4);
    else
        FERRIS_LA_LAUNCH(8);
#undef FERRIS_LA_LAUNCH
}

template <typename T>
int launch_scan(const void* qkv, int ld, int q_off, int k_off, int v_off, float* out, int ldo, float* state,
                float* scratch, const float* decay, const int* seq_q_start, const int* seq_state_slot, int seqs,
                int heads, int dim, int vdim, int silu, int write_state, int seg_len, int segs_max, const RotaryArgs rot,
                cudaStream_t s) {
    if (segs_max <= 1) {
        launch_scan_mode<T, 0>(qkv, ld, q_off, k_off, v_off, out, ldo, state, scratch, decay, seq_q_start, seq_state_slot,
                               seqs, heads, dim, vdim, silu, write_state, seg_len, 1, rot, s);
        FERRIS_LAUNCH_CHECK();
    }
    launch_scan_mode<T, 1>(qkv, ld, q_off, k_off, v_off, out, ldo, state, scratch, decay, seq_q_start, seq_state_slot, seqs,
                           heads, dim, vdim, silu, write_state, seg_len, segs_max, rot, s);
    const size_t per_state = (size_t)heads * vdim * dim;
    ferris_launch(linear_attention_combine_kernel, dim3((unsigned)((per_state + 255) / 256), seqs), dim3(256), 0, s,
                  (const float*)state, scratch, decay, seq_q_start, seq_state_slot, heads, dim, vdim, seg_len);
    launch_scan_mode<T, 2>(qkv, ld, q_off, k_off, v_off, out, ldo, state, scratch, decay, seq_q_start, seq_state_slot, seqs,
                           heads, dim, vdim, silu, write_state, seg_len, segs_max, rot, s);
    FERRIS_LAUNCH_CHECK();
}

}  // namespace

// qkv: rows of ld elements holding q heads at q_off, k heads at k_off (heads x dim each) and v heads at v_off
// (heads x vdim), head by head; out: fp32 [tokens, heads x vdim] rows ldo apart; state: fp32 [slots, heads, vdim, dim];
// decay: fp32 [heads].  The rows of request s are seq_q_start[s] .. seq_q_start[s + 1] - 1, in order.
// segs_max > 1: no request brings more than segs_max * seg_len tokens, and they run as segments of seg_len side by
// side through `scratch`, fp32 [tokens / seg_len + seqs + 1, heads, vdim, dim].
FERRIS_API int ferris_linear_attention(const void* qkv, int ld, int q_off, int k_off, int v_off, int dtype, float* out,
                                       int ldo, float* state, const float* decay, const int* seq_q_start,
                                       const int* seq_state_slot, int seqs, int heads, int dim, int vdim, int silu,
                                       int write_state, int seg_len, int segs_max, float* scratch,
                                       const int* positions, const float* freq, int rotary, int interleaved, float mag,
                                       float k_scale, void* stream) {
    if (seqs <= 0) return FERRIS_OK;
    if (positions && (rotary < 0 || rotary > dim || (rotary & 1) || (rotary > 0 && !freq)))
        FERRIS_REFUSE("linear attention: %d rotated elements of heads of %d", rotary, dim);
    const RotaryArgs rot = {positions, freq, rotary, interleaved, mag, k_scale};
    if (segs_max > 1 && (!scratch || seg_len <= 0)) FERRIS_REFUSE("linear attention: segments need scratch and a length");
    if (seqs > 65535) FERRIS_REFUSE("linear attention: %d requests are more than one launch takes", seqs);
    if (heads <= 0 || dim <= 0 || vdim <= 0 || dim > 256) FERRIS_REFUSE("linear attention: heads=%d dim=%d vdim=%d (dim at most 256)", heads, dim, vdim);
    if (heads > 65535) FERRIS_REFUSE("linear attention: %d heads are more than one launch takes", heads);
    if (!state || !decay) FERRIS_REFUSE("linear attention: no state or no decay");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        return launch_scan<float>(qkv, ld, q_off, k_off, v_off, out, ldo, state, scratch, decay, seq_q_start, seq_state_slot, seqs, heads, dim, vdim, silu, write_state, seg_len, segs_max, rot, s);
    if (dtype == FERRIS_BF16)
        return launch_scan<bf16>(qkv, ld, q_off, k_off, v_off, out, ldo, state, scratch, decay, seq_q_start, seq_state_slot, seqs, heads, dim, vdim, silu, write_state, seg_len, segs_max, rot, s);
    FERRIS_REFUSE("linear attention: unknown dtype %d", dtype);
}

FERRIS_API int ferris_gated_rmsnorm(const float* o, int ldi, const void* g, int ldg, const float* w, void* out, int ldo,
                                    int dtype, int rows, int n, float eps, void* stream) {
    if (rows <= 0) return FERRIS_OK;
    if (n <= 0) FERRIS_REFUSE("gated rmsnorm: %d columns", n);
    const int threads = n >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        ferris_launch(gated_rmsnorm_kernel<float>, dim3(rows), dim3(threads), 0, s, o, ldi, (const float*)g, ldg, w, (float*)out, ldo, n, eps);
    else if (dtype == FERRIS_BF16)
        ferris_launch(gated_rmsnorm_kernel<bf16>, dim3(rows), dim3(threads), 0, s, o, ldi, (const bf16*)g, ldg, w, (bf16*)out, ldo, n, eps);
    else
        FERRIS_REFUSE("gated rmsnorm: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}
