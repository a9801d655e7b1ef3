// A gated linear recurrence per channel (the recurrence inside a recurrent block in the manner of Griffin):
//
//   per block n of the channels (C / blocks neighbouring channels):  r = sigmoid(Ra[n] u_n + ra_n),  i = sigmoid(Ri[n] u_n + ri_n)
//   log a = -c * r * softplus(lam);   a = exp(log a);   s_t = a s_(t-1) + sqrt(1 - a^2) * i * u_t;   out_t = s_t * act(y_t)
//
// u: the step's rows after the short convolution, y: the other branch as projected (act = tanh-form GELU or
// nothing), s: fp32 [slots, C], zero when a request is admitted.  Two kernels.
//
// `rglru_gates`: the two block-diagonal products with fp32 sums, the sigmoids, the decay and the input's factor, all
// fp32: it leaves log a and b = sqrt(1 - a^2) i u per (token, channel).  1 - a^2 is formed as -expm1(2 log a), so that a
// decay close to one keeps its digits.  For the same reason the state moves on as s + (expm1(log a) s + b) and never
// through a itself: a decay of 0.9995 rounded to 24 bits is off by up to 3e-8, a ten-thousandth of what it takes away
// from the state, and where a channel's decay hardly changes from token to token that error has the same sign at
// every step: over a thousand tokens it shows in 32-bit logits.  expm1(log a) s has the relative error of one rounding,
// and the sum rounds at the state's size, sometimes up and sometimes down.  The matrices lie transposed ([blocks, in, out]) so that the threads of a
// block read consecutive weights; eight tokens share one pass over them, and the inputs are cut into four runs that
// four quarters of the block take (their sums added in the runs' order).
//
// `rglru_scan`: s_t = a_t s_(t-1) + b_t is linear in s, so a run of tokens is summed up by (product of its a, kept as
// expm1 of the sum of its log a; its end value from zero) and runs combine.  A block owns SCAN_CH channels of one request and walks its tokens in tiles of
// SEGS x SEG_TOKENS: a thread holds one run of SEG_TOKENS tokens of one channel in registers (all loads of a tile are
// in flight together), forms the run's summary, the summaries meet in shared memory, every thread folds the runs
// before its own onto the tile's incoming value, and then writes its tokens' outputs.  The chain of a tile is
// SEG_TOKENS + SEGS + SEG_TOKENS steps instead of SEGS x SEG_TOKENS.  A step of single tokens is one thread per
// (request, channel); the gates kernel then takes that step itself (STEP): the thread that has formed a token's a and b
// for a channel reads the channel's state, moves it on and writes the gated output, so a and b never reach memory and
// the scan is no launch of its own.
#include <math.h>
#include <mma.h>

#include "common.cuh"

namespace {

constexpr int RG_TOKENS = 8, RG_COLS = 64, RG_PARTS = 4, RG_THREADS = RG_COLS * RG_PARTS;
// eight channels a block (a 32-byte sector of the fp32 rows), 32 runs of eight tokens: a long prompt of a few thousand
// channels fills the SMs, and a tile of 256 tokens costs a chain of 8 + 32 + 8 steps
constexpr int SCAN_CH = 8, SCAN_SEGS = 32, SCAN_SEG_TOKENS = 8, SCAN_THREADS = SCAN_CH * SCAN_SEGS;

__device__ __forceinline__ float sigmoid_r(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float gelu_tanh_r(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// u: [tokens, C] rows ldu apart; wa, wi: [blocks, bs, bs] as [block][input][output]; ba, bi, sp (softplus(lam)): fp32 [C].
// STEP (every request brings one token, row t is request t's): state, slots, the other branch y and the output rows
// are given, a_out and b_out are not.
template <typename T, bool STEP>
__global__ void __launch_bounds__(RG_THREADS) rglru_gates_kernel(const T* u, int ldu, const T* __restrict__ wa,
                                                                 const T* __restrict__ wi, const float* __restrict__ ba,
                                                                 const float* __restrict__ bi, const float* __restrict__ sp,
                                                                 float* __restrict__ a_out, float* __restrict__ b_out,
                                                                 int tokens, int C, int bs, float decay_factor, float* state,
                                                                 const int* __restrict__ seq_state_slot, const T* y, int ldy,
                                                                 T* __restrict__ out, int ldo, int act, int write_state) {
    extern __shared__ float us[];  // [RG_TOKENS][bs], then the parts' sums [RG_PARTS - 1][2][RG_TOKENS][RG_COLS]
    pdl_wait();
    pdl_launch_dependents();
    const int t0 = blockIdx.x * RG_TOKENS, blk = blockIdx.y;
    const int cl = threadIdx.x % RG_COLS, part = threadIdx.x / RG_COLS;
    const int n = blockIdx.z * RG_COLS + cl;
    const int rows = tokens - t0 < RG_TOKENS ? tokens - t0 : RG_TOKENS;
    for (int i = threadIdx.x; i < RG_TOKENS * bs; i += RG_THREADS) {
        const int r = i / bs, k = i - r * bs;
        us[i] = r < rows ? to_float(u[(size_t)(t0 + r) * ldu + (size_t)blk * bs + k]) : 0.0f;
    }
    __syncthreads();
    float acc_a[RG_TOKENS], acc_i[RG_TOKENS];
#pragma unroll
    for (int r = 0; r < RG_TOKENS; ++r) acc_a[r] = 0.0f, acc_i[r] = 0.0f;
    const int per = (bs + RG_PARTS - 1) / RG_PARTS;
    const int k0 = part * per, k1 = min(bs, k0 + per);
    if (n < bs) {
        const T* pa = wa + (size_t)blk * bs * bs + n;
        const T* pi = wi + (size_t)blk * bs * bs + n;
#pragma unroll 4
        for (int k = k0; k < k1; ++k) {
            const float va = to_float(pa[(size_t)k * bs]), vi = to_float(pi[(size_t)k * bs]);
#pragma unroll
            for (int r = 0; r < RG_TOKENS; ++r) {
                const float x = us[r * bs + k];
                acc_a[r] = fmaf(x, va, acc_a[r]), acc_i[r] = fmaf(x, vi, acc_i[r]);
            }
        }
    }
    float* sums = us + RG_TOKENS * bs;
    if (part > 0) {
#pragma unroll
        for (int r = 0; r < RG_TOKENS; ++r) {
            sums[(((part - 1) * 2 + 0) * RG_TOKENS + r) * RG_COLS + cl] = acc_a[r];
            sums[(((part - 1) * 2 + 1) * RG_TOKENS + r) * RG_COLS + cl] = acc_i[r];
        }
    }
    __syncthreads();
    if (part > 0 || n >= bs) return;
    const int c = blk * bs + n;
    const float bias_a = ba[c], bias_i = bi[c], rate = decay_factor * sp[c];
#pragma unroll
    for (int r = 0; r < RG_TOKENS; ++r) {
        if (r >= rows) break;
        float za = acc_a[r], zi = acc_i[r];
#pragma unroll
        for (int p = 0; p < RG_PARTS - 1; ++p) {  // in the runs' order
            za += sums[((p * 2 + 0) * RG_TOKENS + r) * RG_COLS + cl];
            zi += sums[((p * 2 + 1) * RG_TOKENS + r) * RG_COLS + cl];
        }
        const float log_a = -rate * sigmoid_r(za + bias_a);
        const float gate = sigmoid_r(zi + bias_i);
        const float b = sqrtf(-expm1f(2.0f * log_a)) * gate * us[r * bs + n];
        if (STEP) {
            float* S = state + (size_t)seq_state_slot[t0 + r] * C + c;
            const float s_old = *S;
            const float s_new = s_old + fmaf(expm1f(log_a), s_old, b);
            if (write_state) *S = s_new;
            float v = s_new;
            if (y) {
                const float z = to_float(y[(size_t)(t0 + r) * ldy + c]);
                v *= act ? gelu_tanh_r(z) : z;
            }
            out[(size_t)(t0 + r) * ldo + c] = from_float<T>(v);
        } else {
            const size_t at = (size_t)(t0 + r) * C + c;
            a_out[at] = log_a, b_out[at] = b;
        }
    }
}

// The gates of a long step in bf16 on the tensor cores: a block takes 64 tokens x 64 outputs of one gate block for both
// gates; the tokens' inputs of the gate block stand in shared memory (they are also the u of the epilogue), the weights
// are read as they are stored ([block][output][input] is the column-major B operand), sums are fp32 fragments that pass
// through shared memory to the same epilogue as above.  bs a multiple of 64.
constexpr int TG_M = 64, TG_N = 64, TG_THREADS = 128;
__global__ void __launch_bounds__(TG_THREADS) rglru_gates_mma_kernel(const bf16* u, int ldu, const bf16* __restrict__ wa,
                                                                     const bf16* __restrict__ wi,
                                                                     const float* __restrict__ ba,
                                                                     const float* __restrict__ bi,
                                                                     const float* __restrict__ sp, float* __restrict__ a_out,
                                                                     float* __restrict__ b_out, int tokens, int C, int bs,
                                                                     float decay_factor) {
    using namespace nvcuda;
    extern __shared__ __align__(32) uint8_t tg_smem[];
    const int lda = bs + 8;  // elements: sixteen rows (a fragment) are a multiple of 32 bytes, eight rows meet eight bank groups
    bf16* A = reinterpret_cast<bf16*>(tg_smem);
    float* Z = reinterpret_cast<float*>(tg_smem + (((size_t)TG_M * lda * sizeof(bf16) + 31) & ~(size_t)31));  // [2][TG_M][TG_N]
    pdl_wait();
    pdl_launch_dependents();
    const int t0 = blockIdx.x * TG_M, blk = blockIdx.y, n0 = blockIdx.z * TG_N;
    const int warp = threadIdx.x >> 5;
    const int chunks = bs >> 3;  // 16-byte pieces of a row
    for (int i = threadIdx.x; i < TG_M * chunks; i += TG_THREADS) {
        const int r = i / chunks, c8 = (i - r * chunks) << 3;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (t0 + r < tokens) v = *reinterpret_cast<const uint4*>(u + (size_t)(t0 + r) * ldu + (size_t)blk * bs + c8);
        *reinterpret_cast<uint4*>(A + (size_t)r * lda + c8) = v;
    }
    __syncthreads();
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc_a[TG_N / 16], acc_i[TG_N / 16];
#pragma unroll
    for (int j = 0; j < TG_N / 16; ++j) wmma::fill_fragment(acc_a[j], 0.0f), wmma::fill_fragment(acc_i[j], 0.0f);
    const bf16* pa = wa + ((size_t)blk * bs + n0) * bs;
    const bf16* pi = wi + ((size_t)blk * bs + n0) * bs;
#pragma unroll 2
    for (int k0 = 0; k0 < bs; k0 += 16) {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa;
        wmma::load_matrix_sync(fa, A + (size_t)(16 * warp) * lda + k0, lda);
#pragma unroll
        for (int j = 0; j < TG_N / 16; ++j) {
            wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb;
            wmma::load_matrix_sync(fb, pa + (size_t)(16 * j) * bs + k0, bs);
            wmma::mma_sync(acc_a[j], fa, fb, acc_a[j]);
            wmma::load_matrix_sync(fb, pi + (size_t)(16 * j) * bs + k0, bs);
            wmma::mma_sync(acc_i[j], fa, fb, acc_i[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < TG_N / 16; ++j) {
        wmma::store_matrix_sync(Z + (size_t)(16 * warp) * TG_N + 16 * j, acc_a[j], TG_N, wmma::mem_row_major);
        wmma::store_matrix_sync(Z + (size_t)(TG_M + 16 * warp) * TG_N + 16 * j, acc_i[j], TG_N, wmma::mem_row_major);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < TG_M * TG_N; i += TG_THREADS) {
        const int r = i / TG_N, n = i - r * TG_N;
        if (t0 + r >= tokens) break;
        const int c = blk * bs + n0 + n;
        const float log_a = -decay_factor * sp[c] * sigmoid_r(Z[(size_t)r * TG_N + n] + ba[c]);
        const float gate = sigmoid_r(Z[(size_t)(TG_M + r) * TG_N + n] + bi[c]);
        const size_t at = (size_t)(t0 + r) * C + c;
        a_out[at] = log_a;
        b_out[at] = sqrtf(-expm1f(2.0f * log_a)) * gate * to_float(A[(size_t)r * lda + n0 + n]);
    }
}

// a: fp32 [tokens, C], the LOGARITHMS of the decays; b: fp32 [tokens, C]; y: [tokens, C] rows ldy apart (null: the state
// itself is the output); out: rows ldo apart.
template <typename T>
__global__ void __launch_bounds__(SCAN_THREADS) rglru_scan_kernel(const float* a, const float* b, const T* y, int ldy,
                                                                  T* __restrict__ out, int ldo, float* state,
                                                                  const int* __restrict__ seq_q_start,
                                                                  const int* __restrict__ seq_state_slot, int C, int act,
                                                                  int write_state) {
    __shared__ float prod[SCAN_SEGS][SCAN_CH], last[SCAN_SEGS][SCAN_CH], carry[SCAN_CH];
    pdl_wait();
    pdl_launch_dependents();
    const int seq = blockIdx.x;
    const int lane = threadIdx.x % SCAN_CH, seg = threadIdx.x / SCAN_CH;
    const int c = blockIdx.y * SCAN_CH + lane;
    const bool live = c < C;
    const int row0 = seq_q_start[seq], row1 = seq_q_start[seq + 1];
    if (row1 <= row0) return;
    float* S = state + (size_t)seq_state_slot[seq] * C + (live ? c : 0);
    if (seg == 0) carry[lane] = live ? *S : 0.0f;
    constexpr int TILE = SCAN_SEGS * SCAN_SEG_TOKENS;
    for (int t0 = row0; t0 < row1; t0 += TILE) {
        const int first = t0 + seg * SCAN_SEG_TOKENS;
        float av[SCAN_SEG_TOKENS], bv[SCAN_SEG_TOKENS];
#pragma unroll
        for (int j = 0; j < SCAN_SEG_TOKENS; ++j) {
            const bool in = live && first + j < row1;
            av[j] = in ? a[(size_t)(first + j) * C + c] : 0.0f;
            bv[j] = in ? b[(size_t)(first + j) * C + c] : 0.0f;
        }
        float log_p = 0.0f, s = 0.0f;  // the run from zero: the logarithm of its product of decays, and its end value
#pragma unroll
        for (int j = 0; j < SCAN_SEG_TOKENS; ++j) {
            log_p += av[j];
            av[j] = expm1f(av[j]);  // from here on: the decay minus one
            s += fmaf(av[j], s, bv[j]);
        }
        prod[seg][lane] = expm1f(log_p), last[seg][lane] = s;
        __syncthreads();  // also: the carry of the tile before (or the state) is written
        float in_value = carry[lane];
        for (int g = 0; g < seg; ++g) in_value += fmaf(prod[g][lane], in_value, last[g][lane]);
        s = in_value;
#pragma unroll
        for (int j = 0; j < SCAN_SEG_TOKENS; ++j) {
            s += fmaf(av[j], s, bv[j]);
            if (live && first + j < row1) {
                float v = s;
                if (y) {
                    const float z = to_float(y[(size_t)(first + j) * ldy + c]);
                    v *= act ? gelu_tanh_r(z) : z;
                }
                out[(size_t)(first + j) * ldo + c] = from_float<T>(v);
            }
        }
        __syncthreads();  // everyone has read the carry and the summaries
        if (seg == SCAN_SEGS - 1) carry[lane] = s;  // rows beyond the step's end pass the value on (log a = 0, b = 0)
    }
    __syncthreads();
    if (write_state && live && seg == 0) *S = carry[lane];
}

// A step in which every request brings one token: a thread per (request, channel).
template <typename T>
__global__ void __launch_bounds__(256) rglru_scan_single_kernel(const float* a, const float* b, const T* y, int ldy,
                                                                T* __restrict__ out, int ldo, float* state,
                                                                const int* __restrict__ seq_state_slot, int C, int act,
                                                                int write_state) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float* S = state + (size_t)seq_state_slot[t] * C + c;
    const float s_old = *S;
    const float s = s_old + fmaf(expm1f(a[(size_t)t * C + c]), s_old, b[(size_t)t * C + c]);
    if (write_state) *S = s;
    float v = s;
    if (y) {
        const float z = to_float(y[(size_t)t * ldy + c]);
        v *= act ? gelu_tanh_r(z) : z;
    }
    out[(size_t)t * ldo + c] = from_float<T>(v);
}

}  // namespace

// u: [tokens, C] in the activations' type, rows ldu apart; wa, wi: [blocks, C / blocks, C / blocks] in the same type,
// TRANSPOSED ([block][input][output]); ba, bi, sp: fp32 [C] (sp = softplus of the decay's parameter); a_out (log a), b_out: fp32
// [tokens, C]; decay_factor: the constant c of log a = -c r softplus(lam).  With `state` (fp32 [slots, C]; a step in
// which request t brings row t alone): a_out and b_out are not written; the state of slot seq_state_slot[t] moves on
// (if write_state) and out[t] = s * act(y[t]) as in ferris_rglru_scan.
// The tensor-core form of the gates (a long step in bf16, not a step of single tokens): wa, wi as the folder stores them,
// [blocks, output, input]; C / blocks a multiple of 64, rows of u and the matrices on 32 bytes.  Returns
// FERRIS_BAD_ARGUMENT (and says why) for what it does not take.
FERRIS_API int ferris_rglru_gates_mma(const void* u, int ldu, const void* wa, const void* wi, const float* ba,
                                      const float* bi, const float* sp, float* a_out, float* b_out, int tokens, int C,
                                      int blocks, float decay_factor, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (C <= 0 || blocks <= 0 || C % blocks || blocks > 65535) FERRIS_REFUSE("recurrent unit gates: %d channels in %d blocks", C, blocks);
    const int bs = C / blocks;
    if (bs % TG_N || (ldu & 7) || (((uintptr_t)u | (uintptr_t)wa | (uintptr_t)wi) & 31) || !a_out || !b_out)
        FERRIS_REFUSE("recurrent unit gates on tensor cores: blocks of %d channels (a multiple of %d), rows on 32 bytes", bs, TG_N);
    const size_t smem = (((size_t)TG_M * (bs + 8) * sizeof(bf16) + 31) & ~(size_t)31) + (size_t)2 * TG_M * TG_N * sizeof(float);
    if (smem > 200 * 1024) FERRIS_REFUSE("recurrent unit gates on tensor cores: blocks of %d channels are more than shared memory holds", bs);
    int e_ = ferris_allow_dynamic_smem((const void*)rglru_gates_mma_kernel, smem);
    if (e_ != FERRIS_OK) return e_;
    ferris_launch(rglru_gates_mma_kernel, dim3((tokens + TG_M - 1) / TG_M, blocks, bs / TG_N), dim3(TG_THREADS), smem,
                  (cudaStream_t)stream, (const bf16*)u, ldu, (const bf16*)wa, (const bf16*)wi, ba, bi, sp, a_out, b_out, tokens, C,
                  bs, decay_factor);
    FERRIS_LAUNCH_CHECK();
}

FERRIS_API int ferris_rglru_gates(const void* u, int ldu, int dtype, const void* wa, const void* wi, const float* ba,
                                  const float* bi, const float* sp, float* a_out, float* b_out, int tokens, int C,
                                  int blocks, float decay_factor, float* state, const int* seq_state_slot, const void* y,
                                  int ldy, void* out, int ldo, int act, int write_state, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (C <= 0 || blocks <= 0 || C % blocks || blocks > 65535) FERRIS_REFUSE("recurrent unit gates: %d channels in %d blocks", C, blocks);
    const bool step = state != nullptr;  // a step of single tokens: the state moves on here
    if (step ? (!seq_state_slot || !out) : (!a_out || !b_out)) FERRIS_REFUSE("recurrent unit gates: an output is missing");
    const int bs = C / blocks;
    const size_t smem = ((size_t)RG_TOKENS * bs + (size_t)(RG_PARTS - 1) * 2 * RG_TOKENS * RG_COLS) * sizeof(float);
    if (smem > 200 * 1024) FERRIS_REFUSE("recurrent unit gates: blocks of %d channels are more than shared memory holds", bs);
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((tokens + RG_TOKENS - 1) / RG_TOKENS, blocks, (bs + RG_COLS - 1) / RG_COLS), block(RG_THREADS);
    int e_;
#define FERRIS_RG_RUN(T, STEP)                                                                                             \
    do {                                                                                                                   \
        if ((e_ = ferris_allow_dynamic_smem((const void*)rglru_gates_kernel<T, STEP>, smem)) != FERRIS_OK) return e_;      \
        ferris_launch(rglru_gates_kernel<T, STEP>, grid, block, smem, s, (const T*)u, ldu, (const T*)wa, (const T*)wi, ba, \
                      bi, sp, a_out, b_out, tokens, C, bs, decay_factor, state, seq_state_slot, (const T*)y, ldy, (T*)out,  \
                      ldo, act, write_state);                                                                              \
    } while (0)
    if (dtype == FERRIS_F32) {
        if (step) FERRIS_RG_RUN(float, true); else FERRIS_RG_RUN(float, false);
    } else if (dtype == FERRIS_BF16) {
        if (step) FERRIS_RG_RUN(bf16, true); else FERRIS_RG_RUN(bf16, false);
    } else
        FERRIS_REFUSE("recurrent unit gates: unknown dtype %d", dtype);
#undef FERRIS_RG_RUN
    FERRIS_LAUNCH_CHECK();
}

// a (the logarithms of the decays), b: fp32 [tokens, C]; y (may be null), out: the activations' type, rows ldy / ldo apart; state: fp32 [slots, C];
// act: 1 = the tanh form of GELU on y, 0 = y as it is.  single_tokens: every request brings one row (row t of request t).
FERRIS_API int ferris_rglru_scan(const float* a, const float* b, const void* y, int ldy, void* out, int ldo, int dtype,
                                 float* state, const int* seq_q_start, const int* seq_state_slot, int tokens, int seqs,
                                 int C, int act, int write_state, int single_tokens, void* stream) {
    if (tokens <= 0 || seqs <= 0) return FERRIS_OK;
    if (C <= 0 || !a || !b || !state || !out) FERRIS_REFUSE("recurrent unit scan: %d channels, or a tensor is missing", C);
    if (dtype != FERRIS_F32 && dtype != FERRIS_BF16) FERRIS_REFUSE("recurrent unit scan: unknown dtype %d", dtype);
    cudaStream_t s = (cudaStream_t)stream;
    if (single_tokens && tokens == seqs) {
        const int threads = C >= 256 ? 256 : ((C + 31) / 32) * 32;
        const dim3 grid(tokens, (C + threads - 1) / threads);
        if (grid.y > 65535) FERRIS_REFUSE("recurrent unit scan: %d channels are more than one launch takes", C);
        if (dtype == FERRIS_F32)
            ferris_launch(rglru_scan_single_kernel<float>, grid, dim3(threads), 0, s, a, b, (const float*)y, ldy, (float*)out, ldo,
                          state, seq_state_slot, C, act, write_state);
        else
            ferris_launch(rglru_scan_single_kernel<bf16>, grid, dim3(threads), 0, s, a, b, (const bf16*)y, ldy, (bf16*)out, ldo,
                          state, seq_state_slot, C, act, write_state);
        FERRIS_LAUNCH_CHECK();
    }
    const dim3 grid(seqs, (C + SCAN_CH - 1) / SCAN_CH);
    if (grid.y > 65535) FERRIS_REFUSE("recurrent unit scan: %d channels are more than one launch takes", C);
    if (dtype == FERRIS_F32)
        ferris_launch(rglru_scan_kernel<float>, grid, dim3(SCAN_THREADS), 0, s, a, b, (const float*)y, ldy, (float*)out, ldo,
                      state, seq_q_start, seq_state_slot, C, act, write_state);
    else
        ferris_launch(rglru_scan_kernel<bf16>, grid, dim3(SCAN_THREADS), 0, s, a, b, (const bf16*)y, ldy, (bf16*)out, ldo,
                      state, seq_q_start, seq_state_slot, C, act, write_state);
    FERRIS_LAUNCH_CHECK();
}
