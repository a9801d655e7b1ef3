// Recurrences over a state of fixed size whose decay changes from token to token, and what stands around them.
//
//   plain form (a state-space layer in its dual, attention-like reading):
//       S_t = g_t S_(t-1) + k_t (b_t v_t)^T;              o_t = S_t^T q_t + D v_t
//   delta rule (the state is corrected towards v_t along k_t before it is read):
//       S' = g_t S_(t-1);  u = b_t (v_t - S'^T k_t);  S_t = S' + k_t u^T;   o_t = S_t^T q_t
//
// S: [dim, vdim] per (request, head), fp32, zero when the request is admitted; g_t (the decay) and b_t (a step size
// or a gate) are one fp32 number per token and head, made by `recurrence_gates`; q and k come in `qk_heads` heads
// shared by heads / qk_heads value heads each, and may carry one fp32 factor per (token, qk head) each (unit norms:
// the factor is 1 / |x|, formed in fp32 by the gates kernel, so that the vectors themselves are read once as stored).
// The plain form also takes a decay per ROW of the state (per key channel) that changes with every token, given as
// fp32 numbers z per (token, head, row): the row's decay is sigmoid(z)^power = exp(-softplus(-z) * power), formed
// in fp32 where the rows are staged; the decay per head is then left out (gated linear attention).  What is staged is
// the decay MINUS ONE, expm1(-softplus(-z) power), and a row moves on as s + ((decay - 1) s + k u): a decay close to one
// rounded to 24 bits is off by a fixed share of what it takes away, with the same sign at every step where the row's
// decay hardly changes, which over a thousand tokens shows in 32-bit logits; this way only the sum rounds, at the state's
// size, up as often as down.
// That form runs long portions of prompts as segments side by side, because the recurrence is linear in the state
// (S_end = diag(product of the segment's decays) S_start + the segment's own sum): MODE 1 sums every segment but a
// request's last from a zero state into scratch; a kernel of its own multiplies up the rows' decays over each segment
// (as expm1 of the sum of their logarithms); a combine kernel turns those
// into the state at every segment's start; MODE 2 runs every segment from there and writes the outputs, a request's last
// segment also its state.  A segment's place in scratch is (its first row / seg_len) + its request's index in the step,
// which no two segments share.
//
// The columns of S do not depend on one another.  4, 8, 16 or 32 lanes (by the head's size) share a column, each
// holding eight rows of it in registers (rows sub, sub + lanes, ...), and a block of 128 threads owns 32, 16, 8 or 4
// columns of one (request, head): what a token costs is a chain of dependent steps (decay, the product with k summed
// over the lanes, the write), so the chain is kept short and the columns are spread over many blocks.  Sixteen tokens'
// q, k, the block's values, g, b and the factors stand in shared memory at a time, and the next sixteen are on their
// way into registers meanwhile.  The state lies transposed
// in memory, [slot, head, vdim, dim], so that the lanes of a column read consecutive floats.  Tokens of a request are walked in order from its slot, so a step may hold single tokens,
// portions of prompts or both.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int GR_THREADS = 128;
constexpr int GR_KPL = 8;    // rows of the state that a lane holds
constexpr int GR_STAGE = 16;  // tokens in shared memory at a time
constexpr int GR_MAX_DIM = 256;

__device__ __forceinline__ float softplus_g(float v) { return fmaxf(v, 0.0f) + log1pf(expf(-fabsf(v))); }

// decay[t, h] = exp(-exp(A_log[h]) * dt), dt = softplus(a[t, h] + dt_bias[h]);  beta[t, h] = sigmoid(b[t, h]) (kind 0)
// or dt itself (kind 1).  With unit norms: qscale[t, g] = q_mul / sqrt(sum q^2 + eps), kscale[t, g] = 1 / sqrt(sum k^2 + eps).
template <typename T>
__global__ void __launch_bounds__(128) recurrence_gates_kernel(const T* proj, int ld, int a_off, int b_off,
                                                               const float* __restrict__ A_log,
                                                               const float* __restrict__ dt_bias, float* __restrict__ decay,
                                                               float* __restrict__ beta, int beta_kind, const T* qk, int ldqk,
                                                               int q_off, int k_off, int qk_heads, int dim, float unit_eps,
                                                               float q_mul, float* __restrict__ qscale,
                                                               float* __restrict__ kscale, int heads) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const T* row = proj + (size_t)t * ld;
    for (int h = threadIdx.x; h < heads; h += blockDim.x) {
        const float dt = softplus_g(to_float(row[a_off + h]) + dt_bias[h]);
        decay[(size_t)t * heads + h] = expf(-expf(A_log[h]) * dt);
        beta[(size_t)t * heads + h] = beta_kind == 0 ? 1.0f / (1.0f + expf(-to_float(row[b_off + h]))) : dt;
    }
    if (!qscale) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const T* src = qk + (size_t)t * ldqk;
    for (int item = warp; item < 2 * qk_heads; item += warps) {
        const bool is_q = item < qk_heads;
        const int g = is_q ? item : item - qk_heads;
        const T* x = src + (is_q ? q_off : k_off) + (size_t)g * dim;
        float ss = 0.0f;
        for (int i = lane; i < dim; i += 32) {
            const float v = to_float(x[i]);
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss + unit_eps);
        if (lane == 0) {
            if (is_q)
                qscale[(size_t)t * qk_heads + g] = inv * q_mul;
            else
                kscale[(size_t)t * qk_heads + g] = inv;
        }
    }
}

// LANES lanes share a column, GR_KPL rows each: dim <= GR_KPL * LANES.  AHEAD: the next tokens are requested into registers
// while the present ones are worked on (portions of prompts); without it a stage goes straight to shared memory.
template <typename T, int LANES, bool DELTA, bool AHEAD, bool ROWDECAY = false, int MODE = 0>
__global__ void __launch_bounds__(GR_THREADS) gated_recurrence_kernel(
    const T* q, int ldq, const T* k, int ldk, const T* v, int ldv, const float* decay, const float* beta,
    const float* qscale, const float* kscale, const float* __restrict__ skip, float* __restrict__ out, int ldo,
    float* state, const int* __restrict__ seq_q_start, const int* __restrict__ seq_state_slot, int heads, int qk_heads,
    int dim, int vdim, int write_state, const float* row_z, int ldz, float row_power, float q_mul, int seg_len = 0,
    int segs_max = 1, float* scratch_s = nullptr, float* scratch_p = nullptr) {
    constexpr int COLS = GR_THREADS / LANES;  // columns of a block
    constexpr int STAGE = (ROWDECAY && LANES == 32) ? GR_STAGE / 2 : GR_STAGE;  // three staged vectors of 256 rows: fewer tokens
    constexpr int ROWS = GR_KPL * LANES;      // rows of the state that the lanes of a column hold
    constexpr int VP = (STAGE * COLS + GR_THREADS - 1) / GR_THREADS;  // values a thread brings per stage
    __shared__ float qs[STAGE][ROWS];
    __shared__ float ks[STAGE][ROWS];
    __shared__ float vs[STAGE][COLS];
    __shared__ float gs[STAGE], bs[STAGE], fqs[STAGE], fks[STAGE];
    __shared__ float as[ROWDECAY ? STAGE : 1][ROWDECAY ? ROWS : 1];  // the rows' decays minus one of the staged tokens
    pdl_wait();
    pdl_launch_dependents();
    const int seq = MODE ? blockIdx.x / segs_max : blockIdx.x, head = blockIdx.y;
    const int tid = threadIdx.x, sub = tid % LANES, cl = tid / LANES;
    const int col = blockIdx.z * COLS + cl;
    const bool active = col < vdim;
    const int qh = head / (heads / qk_heads);
    int row0 = seq_q_start[seq], row1 = seq_q_start[seq + 1];
    if (row1 <= row0) return;
    // the state lies transposed, [slot, head, vdim, dim]: the lanes of a column read consecutive floats
    float* S = state + (((size_t)seq_state_slot[seq] * heads + head) * vdim + (active ? col : 0)) * (size_t)dim;
    float* S_from = S;
    bool last_segment = true;
    size_t place = 0;
    if (MODE) {  // one segment of the request
        const int first = row0 + (blockIdx.x % segs_max) * seg_len;
        if (first >= row1) return;
        last_segment = first + seg_len >= row1;
        if (MODE == 1 && last_segment) return;  // nobody starts from the end of the last segment
        place = (size_t)(first / seg_len + seq);
        row0 = first, row1 = last_segment ? row1 : first + seg_len;
        S_from = scratch_s + ((place * heads + head) * vdim + (active ? col : 0)) * (size_t)dim;
    }
    float s[GR_KPL];
#pragma unroll
    for (int i = 0; i < GR_KPL; ++i) {
        const int kk = sub + LANES * i;
        s[i] = (MODE != 1 && active && kk < dim) ? S_from[kk] : 0.0f;
    }
    // rows of the staged vectors beyond the head's size stay zero
    for (int i = tid; i < STAGE * ROWS; i += GR_THREADS) {
        (&qs[0][0])[i] = 0.0f, (&ks[0][0])[i] = 0.0f;
        if (ROWDECAY) (&as[0][0])[i] = 0.0f;
    }
    const float d_skip = skip ? skip[head] : 0.0f;
    // A stage's q, k, v and per-token numbers are requested into registers while the stage before it is worked on
    // (the requests of a stage are all in flight together), and go to shared memory when that one is done.
    // (they stay as they were loaded until then: an instruction that touched one would wait for its load)
    T pq[STAGE][2], pk[STAGE][2], pv[VP];
    float pz[ROWDECAY ? STAGE : 1][2];
    float pg = 0.0f, pb = 0.0f, pfq = 1.0f, pfk = 1.0f;
    auto request = [&](int t0) {
#pragma unroll
        for (int r = 0; r < STAGE; ++r) {
            if (t0 + r >= row1) break;  // a single token's block asks for one row
            const size_t row = (size_t)(t0 + r);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int c = tid + j * GR_THREADS;
                if (c < dim) {
                    pq[r][j] = q[row * ldq + (size_t)qh * dim + c];
                    pk[r][j] = k[row * ldk + (size_t)qh * dim + c];
                    if (ROWDECAY) pz[r][j] = row_z[row * ldz + (size_t)head * dim + c];
                }
            }
        }
#pragma unroll
        for (int j = 0; j < VP; ++j) {
            const int e = tid + j * GR_THREADS, r = e / COLS, c = e % COLS;
            const int cc = blockIdx.z * COLS + c;
            pv[j] = from_float<T>(0.0f);
            if (e < STAGE * COLS && t0 + r < row1 && cc < vdim) pv[j] = v[(size_t)(t0 + r) * ldv + (size_t)head * vdim + cc];
        }
        if (tid < STAGE && t0 + tid < row1) {
            const size_t row = (size_t)(t0 + tid);
            pg = decay ? decay[row * heads + head] : 1.0f;
            pb = beta ? beta[row * heads + head] : 1.0f;
            pfq = qscale ? qscale[row * qk_heads + qh] : 1.0f;
            pfk = kscale ? kscale[row * qk_heads + qh] : 1.0f;
        }
    };
    if (AHEAD) request(row0);
    for (int t0 = row0; t0 < row1; t0 += STAGE) {
        const int n = row1 - t0 < STAGE ? row1 - t0 : STAGE;
        __syncthreads();  // the tokens before are done with (and the zeroing above has landed)
        if (!AHEAD) {  // a few tokens a request (a step of single tokens): straight into shared memory
            for (int i = tid; i < n * dim; i += GR_THREADS) {
                const int r = i / dim, c = i - r * dim;
                const size_t row = (size_t)(t0 + r);
                qs[r][c] = to_float(q[row * ldq + (size_t)qh * dim + c]);
                ks[r][c] = to_float(k[row * ldk + (size_t)qh * dim + c]);
                if (ROWDECAY) as[r][c] = expm1f(-softplus_g(-row_z[row * ldz + (size_t)head * dim + c]) * row_power);
            }
            for (int i = tid; i < n * COLS; i += GR_THREADS) {
                const int r = i / COLS, c = i - r * COLS;
                const int cc = blockIdx.z * COLS + c;
                vs[r][c] = cc < vdim ? to_float(v[(size_t)(t0 + r) * ldv + (size_t)head * vdim + cc]) : 0.0f;
            }
            if (tid < n) {
                const size_t row = (size_t)(t0 + tid);
                gs[tid] = decay ? decay[row * heads + head] : 1.0f;
                bs[tid] = beta ? beta[row * heads + head] : 1.0f;
                fqs[tid] = qscale ? qscale[row * qk_heads + qh] : 1.0f;
                fks[tid] = kscale ? kscale[row * qk_heads + qh] : 1.0f;
            }
        } else {
#pragma unroll
        for (int r = 0; r < STAGE; ++r) {
            if (r >= n) break;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int c = tid + j * GR_THREADS;
                if (c < dim) {
                    qs[r][c] = to_float(pq[r][j]), ks[r][c] = to_float(pk[r][j]);
                    if (ROWDECAY) as[r][c] = expm1f(-softplus_g(-pz[r][j]) * row_power);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < VP; ++j) {
            const int e = tid + j * GR_THREADS;
            if (e < n * COLS) (&vs[0][0])[e] = to_float(pv[j]);
        }
        if (tid < STAGE) gs[tid] = pg, bs[tid] = pb, fqs[tid] = pfq, fks[tid] = pfk;
        }
        __syncthreads();
        if (AHEAD && t0 + STAGE < row1) request(t0 + STAGE);
        for (int r = 0; r < n; ++r) {
            const float g = gs[r], b = bs[r], vv = vs[r][cl], fq = fqs[r], fk = fks[r];
            float kr[GR_KPL], qr[GR_KPL];
#pragma unroll
            for (int i = 0; i < GR_KPL; ++i) kr[i] = ks[r][sub + LANES * i], qr[i] = qs[r][sub + LANES * i];
            // the factors of q and k are one number a token each: they multiply the sums, not the vectors
            float uk, od0 = 0.0f, od1 = 0.0f;
            if (DELTA) {
                float d0 = 0.0f, d1 = 0.0f;  // two chains, so that the sum waits for half as many dependent FMAs
#pragma unroll
                for (int i = 0; i < GR_KPL; i += 2) {
                    s[i] *= g, s[i + 1] *= g;
                    d0 = fmaf(s[i], kr[i], d0), d1 = fmaf(s[i + 1], kr[i + 1], d1);
                }
                float dot = d0 + d1;
#pragma unroll
                for (int o = 1; o < LANES; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                uk = (b * (vv - fk * dot)) * fk;
#pragma unroll
                for (int i = 0; i < GR_KPL; i += 2) {
                    s[i] = fmaf(kr[i], uk, s[i]), s[i + 1] = fmaf(kr[i + 1], uk, s[i + 1]);
                    od0 = fmaf(s[i], qr[i], od0), od1 = fmaf(s[i + 1], qr[i + 1], od1);
                }
            } else {
                uk = (b * vv) * fk;
#pragma unroll
                for (int i = 0; i < GR_KPL; i += 2) {
                    if (ROWDECAY) {  // s + ((decay - 1) s + k u)
                        s[i] += fmaf(as[r][sub + LANES * i], s[i], kr[i] * uk);
                        s[i + 1] += fmaf(as[r][sub + LANES * (i + 1)], s[i + 1], kr[i + 1] * uk);
                    } else {
                        s[i] = fmaf(g, s[i], kr[i] * uk), s[i + 1] = fmaf(g, s[i + 1], kr[i + 1] * uk);
                    }
                    od0 = fmaf(s[i], qr[i], od0), od1 = fmaf(s[i + 1], qr[i + 1], od1);
                }
            }
            float od = od0 + od1;
#pragma unroll
            for (int o = 1; o < LANES; o <<= 1) od += __shfl_xor_sync(0xffffffffu, od, o);
            if (MODE != 1 && sub == 0 && active)
                out[(size_t)(t0 + r) * ldo + (size_t)head * vdim + col] = fmaf(d_skip, vv, (fq * q_mul) * od);
        }
    }
    if (MODE == 1) {  // the segment's own sum
#pragma unroll
        for (int i = 0; i < GR_KPL; ++i) {
            const int kk = sub + LANES * i;
            if (active && kk < dim) S_from[kk] = s[i];
        }
        return;
    }
    if (write_state && active && last_segment) {
#pragma unroll
        for (int i = 0; i < GR_KPL; ++i) {
            const int kk = sub + LANES * i;
            if (kk < dim) S[kk] = s[i];
        }
    }
}

// The product of every row's decays over a segment, minus one: expm1 of the sum of the logarithms -softplus(-z) power.
// A block per (request, segment) and head, a thread per row; the last segment of a request has no use for it.
__global__ void __launch_bounds__(256) row_decay_products_kernel(const float* row_z, int ldz, float row_power,
                                                                 float* __restrict__ scratch_p,
                                                                 const int* __restrict__ seq_q_start, int heads, int dim,
                                                                 int seg_len, int segs_max) {
    pdl_wait();
    pdl_launch_dependents();
    const int seq = blockIdx.x / segs_max, head = blockIdx.y;
    const int row0 = seq_q_start[seq], row1 = seq_q_start[seq + 1];
    const int first = row0 + (blockIdx.x % segs_max) * seg_len;
    if (first >= row1 || first + seg_len >= row1) return;
    const size_t place = (size_t)(first / seg_len + seq);
    for (int r = threadIdx.x; r < dim; r += blockDim.x) {
        float sum = 0.0f;
        for (int t = first; t < first + seg_len; ++t) sum -= softplus_g(-row_z[(size_t)t * ldz + (size_t)head * dim + r]) * row_power;
        scratch_p[(place * heads + head) * (size_t)dim + r] = expm1f(sum);
    }
}

// Between the two passes over segments: scratch_s holds every segment's own sum (but the last one's of a request);
// afterwards it holds the state at every segment's start: S_start(0) = the request's state, S_start(n + 1) =
// diag(products of segment n's decays) S_start(n) + sum(n), the products given minus one.  A thread per element of a
// (request, head)'s state.
__global__ void __launch_bounds__(256) row_decay_combine_kernel(float* scratch_s, const float* scratch_p, const float* state,
                                                                const int* __restrict__ seq_q_start,
                                                                const int* __restrict__ seq_state_slot, int heads, int dim,
                                                                int vdim, int seg_len) {
    pdl_wait();
    pdl_launch_dependents();
    const int seq = blockIdx.x, head = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;  // column * dim + row
    if (e >= vdim * dim) return;
    const int row = e % dim;
    const int row0 = seq_q_start[seq], row1 = seq_q_start[seq + 1];
    if (row1 <= row0) return;
    float s = state[((size_t)seq_state_slot[seq] * heads + head) * (size_t)vdim * dim + e];
    for (int first = row0; first < row1; first += seg_len) {
        const size_t place = (size_t)(first / seg_len + seq);
        float* at = scratch_s + (place * heads + head) * (size_t)vdim * dim + e;
        const bool last = first + seg_len >= row1;
        const float own = last ? 0.0f : *at;
        *at = s;
        if (last) break;
        s += fmaf(scratch_p[(place * heads + head) * (size_t)dim + row], s, own);
    }
}

// out = norm(o [* a(gate)]) * w [* a(gate)]: every `group` consecutive columns of a row divided by their own
// sqrt(mean(.^2) + eps), times w[column % wlen]; the gate (a = sigmoid or SiLU) multiplies before the norm
// (gate_first) or after it.  o fp32; gate and out in the activations' type.  A block per row; a warp per group, or
// the whole block for each group in turn where groups are long.
template <typename T>
__global__ void __launch_bounds__(256) gated_group_norm_kernel(const float* o, int ldi, const T* gate, int ldg,
                                                               const float* __restrict__ w, int wlen, T* __restrict__ out,
                                                               int ldo, int n, int group, float eps, int gate_kind,
                                                               int gate_first) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const float* orow = o + (size_t)t * ldi;
    const T* grow = gate ? gate + (size_t)t * ldg : nullptr;
    T* dst = out + (size_t)t * ldo;
    if (group >= 512) {  // few, long groups: the whole block takes them in turn
        __shared__ float scratch[33];
        for (int base = 0; base < n; base += group) {
            float ss = 0.0f;
            for (int i = threadIdx.x; i < group; i += blockDim.x) {
                float val = orow[base + i];
                if (grow && gate_first) {
                    const float z = to_float(grow[base + i]);
                    const float sg = 1.0f / (1.0f + expf(-z));
                    val *= gate_kind == 1 ? z * sg : sg;
                }
                ss = fmaf(val, val, ss);
            }
            ss = block_sum(ss, scratch);
            const float inv = 1.0f / sqrtf(ss / (float)group + eps);
            for (int i = threadIdx.x; i < group; i += blockDim.x) {
                float val = orow[base + i];
                float gv = 1.0f;
                if (grow) {
                    const float z = to_float(grow[base + i]);
                    const float sg = 1.0f / (1.0f + expf(-z));
                    gv = gate_kind == 1 ? z * sg : sg;
                }
                if (gate_first) val *= gv;
                float y = (val * inv) * w[(base + i) % wlen];
                if (!gate_first) y *= gv;
                dst[base + i] = from_float<T>(y);
            }
        }
        return;
    }
    for (int gi = warp; gi * group < n; gi += warps) {
        const int base = gi * group;
        float ss = 0.0f;
        for (int i = lane; i < group; i += 32) {
            float val = orow[base + i];
            if (grow && gate_first) {
                const float z = to_float(grow[base + i]);
                const float sg = 1.0f / (1.0f + expf(-z));
                val *= gate_kind == 1 ? z * sg : sg;
            }
            ss = fmaf(val, val, ss);
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)group + eps);
        for (int i = lane; i < group; i += 32) {
            float val = orow[base + i];
            float gv = 1.0f;
            if (grow) {
                const float z = to_float(grow[base + i]);
                const float sg = 1.0f / (1.0f + expf(-z));
                gv = gate_kind == 1 ? z * sg : sg;
            }
            if (gate_first) val *= gv;
            float y = (val * inv) * w[(base + i) % wlen];
            if (!gate_first) y *= gv;
            dst[base + i] = from_float<T>(y);
        }
    }
}

template <typename T, bool DELTA, bool AHEAD, bool ROWDECAY = false, int MODE = 0>
int launch_recurrence(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, const float* decay,
                      const float* beta, const float* qscale, const float* kscale, const float* skip, float* out, int ldo,
                      float* state, const int* seq_q_start, const int* seq_state_slot, int seqs, int heads, int qk_heads,
                      int dim, int vdim, int write_state, cudaStream_t s, const float* row_z = nullptr, int ldz = 0,
                      float row_power = 1.0f, float q_mul = 1.0f, int seg_len = 0, int segs_max = 1,
                      float* scratch_s = nullptr, float* scratch_p = nullptr) {
    const dim3 block(GR_THREADS);
#define FERRIS_GR_LAUNCH(LANES)                                                                                         \
    ferris_launch(gated_recurrence_kernel<T, LANES, DELTA, AHEAD, ROWDECAY, MODE>,                                    \
                  dim3(seqs * segs_max, heads, (vdim + GR_THREADS / LANES - 1) / (GR_THREADS / LANES)), block, 0, s,   \
                  (const T*)q, ldq, (const T*)k, ldk, (const T*)v, ldv, decay, beta, qscale, kscale, skip, out, ldo,    \
                  state, seq_q_start, seq_state_slot, heads, qk_heads, dim, vdim, write_state, row_z, ldz, row_power,   \
                  q_mul, seg_len, segs_max, scratch_s, scratch_p)
    if (dim <= 32)
        FERRIS_GR_LAUNCH(4);
    else if (dim <= 64)
        FERRIS_GR_LAUNCH(8);
    else if (dim <= 128)
        FERRIS_GR_LAUNCH(16);
    else
        FERRIS_GR_LAUNCH(32);
#undef FERRIS_GR_LAUNCH
    FERRIS_LAUNCH_CHECK();
}

}  // namespace

// proj: [tokens, ld] rows holding a (heads columns from a_off) and, for beta_kind 0, b (heads columns from b_off).
// qk: rows holding q and k heads (qk_heads x dim each) from q_off / k_off; qscale / kscale (null: no unit norms):
// fp32 [tokens, qk_heads].  decay, beta: fp32 [tokens, heads].
FERRIS_API int ferris_recurrence_gates(const void* proj, int ld, int dtype, int a_off, int b_off, const float* A_log,
                                       const float* dt_bias, float* decay, float* beta, int beta_kind, const void* qk,
                                       int ldqk, int q_off, int k_off, int qk_heads, int dim, float unit_eps, float q_mul,
                                       float* qscale, float* kscale, int tokens, int heads, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (heads <= 0 || !A_log || !dt_bias || !decay || !beta) FERRIS_REFUSE("recurrence gates: %d heads, or a table is missing", heads);
    if (beta_kind != 0 && beta_kind != 1) FERRIS_REFUSE("recurrence gates: unknown kind %d of the second number", beta_kind);
    if ((qscale == nullptr) != (kscale == nullptr)) FERRIS_REFUSE("recurrence gates: unit norms of q and k go together");
    if (qscale && (!qk || qk_heads <= 0 || dim <= 0)) FERRIS_REFUSE("recurrence gates: unit norms of %d heads of %d", qk_heads, dim);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        ferris_launch(recurrence_gates_kernel<float>, dim3(tokens), dim3(128), 0, s, (const float*)proj, ld, a_off, b_off,
                      A_log, dt_bias, decay, beta, beta_kind, (const float*)qk, ldqk, q_off, k_off, qk_heads, dim, unit_eps,
                      q_mul, qscale, kscale, heads);
    else if (dtype == FERRIS_BF16)
        ferris_launch(recurrence_gates_kernel<bf16>, dim3(tokens), dim3(128), 0, s, (const bf16*)proj, ld, a_off, b_off,
                      A_log, dt_bias, decay, beta, beta_kind, (const bf16*)qk, ldqk, q_off, k_off, qk_heads, dim, unit_eps,
                      q_mul, qscale, kscale, heads);
    else
        FERRIS_REFUSE("recurrence gates: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}

// q, k: [tokens, qk_heads x dim] from their first column, rows ldq / ldk apart; v: [tokens, heads x vdim], rows ldv apart;
// out: fp32 [tokens, heads x vdim]; state: fp32 [slots, heads, vdim, dim] (transposed); skip: fp32 [heads] or null.
FERRIS_API int ferris_gated_recurrence(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, int dtype,
                                       const float* decay, const float* beta, const float* qscale, const float* kscale,
                                       const float* skip, float* out, int ldo, float* state, const int* seq_q_start,
                                       const int* seq_state_slot, int seqs, int heads, int qk_heads, int dim, int vdim,
                                       int delta_rule, int write_state, int longest, void* stream) {
    if (seqs <= 0) return FERRIS_OK;
    if (heads <= 0 || qk_heads <= 0 || heads % qk_heads) FERRIS_REFUSE("recurrence: %d heads over %d q/k heads", heads, qk_heads);
    if (dim <= 0 || dim > GR_MAX_DIM || vdim <= 0) FERRIS_REFUSE("recurrence: heads of %d x %d (at most %d rows)", dim, vdim, GR_MAX_DIM);
    if (heads > 65535 || (vdim + 3) / 4 > 65535) FERRIS_REFUSE("recurrence: too many heads or columns for one launch");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype != FERRIS_F32 && dtype != FERRIS_BF16) FERRIS_REFUSE("recurrence: unknown dtype %d", dtype);
    const bool ahead = longest > GR_STAGE;  // `longest`: the most tokens a request brings (0: not known)
#define FERRIS_GR_GO(T, D, A)                                                                                                \
    return launch_recurrence<T, D, A>(q, ldq, k, ldk, v, ldv, decay, beta, qscale, kscale, skip, out, ldo, state, seq_q_start, \
                                      seq_state_slot, seqs, heads, qk_heads, dim, vdim, write_state, s)
    if (dtype == FERRIS_F32) {
        if (delta_rule) { if (ahead) FERRIS_GR_GO(float, true, true); else FERRIS_GR_GO(float, true, false); }
        if (ahead) FERRIS_GR_GO(float, false, true); else FERRIS_GR_GO(float, false, false);
    }
    if (delta_rule) { if (ahead) FERRIS_GR_GO(bf16, true, true); else FERRIS_GR_GO(bf16, true, false); }
    if (ahead) FERRIS_GR_GO(bf16, false, true); else FERRIS_GR_GO(bf16, false, false);
#undef FERRIS_GR_GO
}

// The plain form with a decay per row of the state: row_z fp32 [tokens, heads x dim], rows ldz apart; the decay of
// row r of head h at token t is sigmoid(row_z[t, h, r])^row_power.  q and k come in `heads` heads; out = q_mul S^T q.
// segs_max > 1: no request brings more than segs_max * seg_len tokens, and they run as segments of seg_len side by side;
// scratch_s: fp32 [(tokens / seg_len + seqs + 1), heads, vdim, dim], scratch_p: fp32 [the same places, heads, dim].
FERRIS_API int ferris_row_decay_recurrence(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, int dtype,
                                           const float* row_z, int ldz, float row_power, float q_mul, float* out, int ldo,
                                           float* state, const int* seq_q_start, const int* seq_state_slot, int seqs,
                                           int heads, int dim, int vdim, int write_state, int longest, int seg_len,
                                           int segs_max, float* scratch_s, float* scratch_p, void* stream) {
    if (seqs <= 0) return FERRIS_OK;
    if (heads <= 0 || !row_z) FERRIS_REFUSE("row-decay recurrence: %d heads, or no decays", heads);
    if (dim <= 0 || dim > GR_MAX_DIM || vdim <= 0) FERRIS_REFUSE("row-decay recurrence: heads of %d x %d (at most %d rows)", dim, vdim, GR_MAX_DIM);
    if (heads > 65535 || (vdim + 3) / 4 > 65535) FERRIS_REFUSE("row-decay recurrence: too many heads or columns for one launch");
    if (dtype != FERRIS_F32 && dtype != FERRIS_BF16) FERRIS_REFUSE("row-decay recurrence: unknown dtype %d", dtype);
    if (segs_max > 1 && (!scratch_s || !scratch_p || seg_len <= 0)) FERRIS_REFUSE("row-decay recurrence: segments need scratch and a length");
    cudaStream_t s = (cudaStream_t)stream;
    const bool ahead = longest > GR_STAGE;
#define FERRIS_RD_GO(T, A, M)                                                                                                \
    launch_recurrence<T, false, A, true, M>(q, ldq, k, ldk, v, ldv, nullptr, nullptr, nullptr, nullptr, nullptr, out, ldo,    \
                                            state, seq_q_start, seq_state_slot, seqs, heads, heads, dim, vdim, write_state,  \
                                            s, row_z, ldz, row_power, q_mul, seg_len, M ? segs_max : 1, scratch_s, scratch_p)
    if (segs_max > 1) {  // segments side by side: sums, carry, outputs.  Many blocks hide one another's loads, so a stage
        // goes straight to shared memory: the form that requests the next tokens into registers holds four blocks an SM
        int rc = dtype == FERRIS_F32 ? FERRIS_RD_GO(float, false, 1) : FERRIS_RD_GO(bf16, false, 1);
        if (rc != FERRIS_OK) return rc;
        ferris_launch(row_decay_products_kernel, dim3(seqs * segs_max, heads), dim3(dim >= 128 ? 256 : 64), 0, s, row_z, ldz,
                      row_power, scratch_p, seq_q_start, heads, dim, seg_len, segs_max);
        const int elems = vdim * dim;
        ferris_launch(row_decay_combine_kernel, dim3(seqs, heads, (elems + 255) / 256), dim3(256), 0, s, scratch_s,
                      (const float*)scratch_p, (const float*)state, seq_q_start, seq_state_slot, heads, dim, vdim, seg_len);
        return dtype == FERRIS_F32 ? FERRIS_RD_GO(float, false, 2) : FERRIS_RD_GO(bf16, false, 2);
    }
    if (dtype == FERRIS_F32) return ahead ? FERRIS_RD_GO(float, true, 0) : FERRIS_RD_GO(float, false, 0);
    return ahead ? FERRIS_RD_GO(bf16, true, 0) : FERRIS_RD_GO(bf16, false, 0);
#undef FERRIS_RD_GO
}

// o: fp32 [rows, n]; gate (may be null), out: the activations' type; w: fp32 [wlen], wlen dividing n.
FERRIS_API int ferris_gated_group_norm(const float* o, int ldi, const void* gate, int ldg, const float* w, int wlen,
                                       void* out, int ldo, int dtype, int rows, int n, int group, float eps,
                                       int gate_kind, int gate_first, void* stream) {
    if (rows <= 0) return FERRIS_OK;
    if (n <= 0 || group <= 0 || n % group || wlen <= 0 || n % wlen) FERRIS_REFUSE("gated group norm: %d columns in groups of %d, %d weights", n, group, wlen);
    if (gate_kind != 0 && gate_kind != 1) FERRIS_REFUSE("gated group norm: unknown gate %d", gate_kind);
    const int groups = n / group;
    const int threads = group >= 512 ? 256 : (groups >= 8 ? 256 : (groups >= 4 ? 128 : (groups >= 2 ? 64 : 32)));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        ferris_launch(gated_group_norm_kernel<float>, dim3(rows), dim3(threads), 0, s, o, ldi, (const float*)gate, ldg, w, wlen, (float*)out, ldo, n, group, eps, gate_kind, gate_first);
    else if (dtype == FERRIS_BF16)
        ferris_launch(gated_group_norm_kernel<bf16>, dim3(rows), dim3(threads), 0, s, o, ldi, (const bf16*)gate, ldg, w, wlen, (bf16*)out, ldo, n, group, eps, gate_kind, gate_first);
    else
        FERRIS_REFUSE("gated group norm: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}
