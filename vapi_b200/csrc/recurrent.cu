// Mixers that carry a state of fixed size from token to token: a short causal convolution
// per channel with SiLU, the gated delta rule, and the selective state-space recurrence of
// Mamba-2.  A request's state lives in its slot, in float: first the convolution's last L-1
// inputs [L-1, channels], then the recurrent matrices [heads, rows, cols].  Memory is never
// cleared: a sequence whose first token of the step sits at position 0 starts from zeros
// whatever its slot holds.  Everything that enters a recurrence (decays, step sizes, gates,
// unit norms, the state itself) is float; the projections and convolutions that feed it may be
// bfloat16.
#include "common.cuh"

using namespace vapi;

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

// ---------------------------------------------------------------------------------------------
// out[t, c] = silu(bias[c] + sum_j taps[j, c] * x[t - (L-1) + j, c]),  taps oldest first, the
// last one the current token's; inputs before position 0 are zero; inputs before the step come
// from the state, which is then moved on to the step's end.
//
// The first blocks own (sequence, channel) pairs: they read the old state, compute the first
// L-1 tokens of the sequence's portion (the only ones that need it) and write the new state, so
// nothing reads a state that another thread has already replaced.  The other blocks own
// (token, channel) pairs whose whole reach lies inside the portion.
constexpr int CONV_MAX_L = 8;

template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ taps,
                                        const float* __restrict__ bias, float* __restrict__ state,
                                        long long slot_stride, const int* __restrict__ state_slots,
                                        const int* __restrict__ tok_seq, const int* __restrict__ cu_q,
                                        const int* __restrict__ positions, T* __restrict__ out, int n, int num_seqs,
                                        int channels, int L, int num_slots, int head_blocks, int* __restrict__ status) {
    pdl_trigger();
    if ((int)blockIdx.x < head_blocks) {
        const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
        if (item >= (long long)num_seqs * channels) {
            pdl_wait();
            return;
        }
        const int s = (int)(item / channels), c = (int)(item - (long long)s * channels);
        const int q0 = cu_q[s], qlen = cu_q[s + 1] - q0;
        if (qlen <= 0) {
            pdl_wait();
            return;
        }
        const int slot = state_slots[s], start = positions[q0];
        float w[CONV_MAX_L];
        for (int j = 0; j < L; ++j) w[j] = taps[(size_t)j * channels + c];
        const float b = bias ? bias[c] : 0.f;
        if (slot < 0 || slot >= num_slots) {
            if (status) atomicExch(status, 3);
            pdl_wait();
            return;
        }
        float* st = state + (size_t)slot * slot_stride;
        pdl_wait();
        // hist[r] = input at position start - (L-1) + r, r = 0 .. L-2
        float hist[CONV_MAX_L];
        for (int r = 0; r < L - 1; ++r) {
            const int pos = start - (L - 1) + r;
            hist[r] = pos >= 0 ? st[(size_t)r * channels + c] : 0.f;
        }
        const int head = min(qlen, L - 1);
        // inputs of the first tokens of the portion follow the history
        float win[2 * CONV_MAX_L];
        for (int r = 0; r < L - 1; ++r) win[r] = hist[r];
        for (int i = 0; i < head; ++i) win[L - 1 + i] = to_f32(x[(size_t)(q0 + i) * x_stride + c]);
        for (int i = 0; i < head; ++i) {
            float acc = b;
            for (int j = 0; j < L; ++j) acc = fmaf(w[j], win[i + j], acc);
            out[(size_t)(q0 + i) * channels + c] = from_f32<T>(silu_f(acc));
        }
        // the new state: the last L-1 inputs before position start + qlen
        for (int r = 0; r < L - 1; ++r) {
            const int back = (L - 1) - r;                 // this entry is the input at end - back
            float v;
            if (back <= qlen) v = to_f32(x[(size_t)(q0 + qlen - back) * x_stride + c]);
            else v = hist[r + qlen];                      // still an input from before the step
            st[(size_t)r * channels + c] = v;
        }
        return;
    }
    const long long item = (long long)(blockIdx.x - head_blocks) * blockDim.x + threadIdx.x;
    pdl_wait();
    if (item >= (long long)n * channels) return;
    const int t = (int)(item / channels), c = (int)(item - (long long)t * channels);
    const int s = tok_seq[t];
    const int i = t - cu_q[s];
    if (i < L - 1) return;                                 // a head token: the other blocks' work
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < L; ++j)
        acc = fmaf(taps[(size_t)j * channels + c], to_f32(x[(size_t)(t - (L - 1) + j) * x_stride + c]), acc);
    out[(size_t)t * channels + c] = from_f32<T>(silu_f(acc));
}

VAPI_EXPORT int vapi_causal_conv_silu(const void* x, long long x_stride, int dtype, const float* taps, const float* bias,
                                      float* state, long long slot_stride, const int* state_slots, const int* tok_seq,
                                      const int* cu_q, const int* positions, void* out, int n, int num_seqs,
                                      int channels, int L, int num_slots, int max_q, int* status, cudaStream_t stream) {
    if (n <= 0 || num_seqs <= 0) return 0;
    if (channels <= 0 || L < 1 || L > CONV_MAX_L) return fail(-1, "causal_conv_silu: %d channels, %d taps", channels, L);
    if (L > 1 && !state) return fail(-1, "causal_conv_silu: a convolution of %d taps needs a state", L);
    const int threads = 128;
    const int head_blocks = L > 1 ? (int)(((long long)num_seqs * channels + threads - 1) / threads) : 0;
    const int body_blocks = max_q > L - 1 ? (int)(((long long)n * channels + threads - 1) / threads) : 0;
    if (head_blocks + body_blocks == 0) return 0;
    cudaError_t e;
    if (dtype == VAPI_F32)
        e = launch(causal_conv_silu_kernel<float>, head_blocks + body_blocks, threads, 0, stream, (const float*)x, x_stride, taps,
                   bias, state, slot_stride, state_slots, tok_seq, cu_q, positions, (float*)out, n, num_seqs, channels, L,
                   num_slots, head_blocks, status);
    else if (dtype == VAPI_BF16)
        e = launch(causal_conv_silu_kernel<__nv_bfloat16>, head_blocks + body_blocks, threads, 0, stream, (const __nv_bfloat16*)x,
                   x_stride, taps, bias, state, slot_stride, state_slots, tok_seq, cu_q, positions, (__nv_bfloat16*)out, n,
                   num_seqs, channels, L, num_slots, head_blocks, status);
    else
        return fail(-2, "causal_conv_silu: unsupported dtype %d", dtype);
    return check_launch("causal_conv_silu", e);
}

// ---------------------------------------------------------------------------------------------
// The two recurrences share one decomposition.  The state of a head is a matrix S [rows, cols]
// (delta rule: key size x value size; state space: state size x head size).  A block owns one
// (sequence, head) and a slice of the columns and walks the sequence's tokens in order.  A column
// is shared by LPC neighbouring lanes, each holding RT consecutive rows of it in registers
// (RT * LPC >= rows); sums over the rows end with log2(LPC) shuffles.  The next token's inputs
// are requested before this token's arithmetic.
constexpr int REC_THREADS = 128;

template <int LPC>
__device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
    for (int o = LPC >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Gated delta rule.  Per token, with k and q made unit vectors (q also times rows^-1/2):
//   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//   beta = sigmoid(b),  g = exp(-exp(A_log) * softplus(a + dt_bias)).
// qkv [n, *]: q heads [nkv, rows], k heads [nkv, rows], v heads [nh, cols] at the given column
// offsets of a row of `qkv_stride` elements; ab [n, *]: a [nh] then b [nh] at `ab` with its stride.
template <typename T, int RT, int LPC>
__global__ void __launch_bounds__(REC_THREADS)
gated_delta_kernel(const T* __restrict__ qkv, long long qkv_stride, int q_off, int k_off, int v_off,
                   const T* __restrict__ ab, long long ab_stride, const float* __restrict__ A_log,
                   const float* __restrict__ dt_bias, float* __restrict__ state, long long slot_stride,
                   const int* __restrict__ state_slots, const int* __restrict__ cu_q,
                   const int* __restrict__ positions, float* __restrict__ out, int nh, int nkv, int rows, int cols,
                   int num_slots, float norm_eps, int* __restrict__ status) {
    constexpr int CPB = REC_THREADS / LPC;              // columns per block
    const int s = blockIdx.z, h = blockIdx.y;
    const int col = blockIdx.x * CPB + threadIdx.x / LPC;
    const int sl = threadIdx.x % LPC;
    const int r0 = sl * RT;
    const int g = h / (nh / nkv);
    const bool col_ok = col < cols;
    pdl_trigger();
    const int t0 = cu_q[s], qlen = cu_q[s + 1] - t0;
    if (qlen <= 0) return;
    const int slot = state_slots[s];
    if (slot < 0 || slot >= num_slots) {
        if (status) atomicExch(status, 3);
        return;
    }
    const float decay_rate = expf(A_log[h]);
    const float bias = dt_bias[h];
    const float q_scale = rsqrtf((float)rows);
    float* S_glob = state + (size_t)slot * slot_stride + ((size_t)h * rows) * cols;
    const bool fresh = positions[t0] == 0;
    pdl_wait();
    float S[RT];
#pragma unroll
    for (int r = 0; r < RT; ++r)
        S[r] = (!fresh && col_ok && r0 + r < rows) ? S_glob[(size_t)(r0 + r) * cols + col] : 0.f;

    float kc[RT], qc[RT], vc, ac, bc;
    auto fetch = [&](int t, float (&kk)[RT], float (&qq)[RT], float& vv, float& aa, float& bb) {
        const T* row = qkv + (size_t)t * qkv_stride;
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            const bool ok = r0 + r < rows;
            kk[r] = ok ? to_f32(row[k_off + g * rows + r0 + r]) : 0.f;
            qq[r] = ok ? to_f32(row[q_off + g * rows + r0 + r]) : 0.f;
        }
        vv = col_ok ? to_f32(row[v_off + h * cols + col]) : 0.f;
        aa = to_f32(ab[(size_t)t * ab_stride + h]);
        bb = to_f32(ab[(size_t)t * ab_stride + nh + h]);
    };
    fetch(t0, kc, qc, vc, ac, bc);
    for (int i = 0; i < qlen; ++i) {
        float kn[RT], qn[RT], vn = 0.f, an = 0.f, bn = 0.f;
        if (i + 1 < qlen) fetch(t0 + i + 1, kn, qn, vn, an, bn);
        float ssk = 0.f, ssq = 0.f;
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            ssk = fmaf(kc[r], kc[r], ssk);
            ssq = fmaf(qc[r], qc[r], ssq);
        }
        ssk = lanes_sum<LPC>(ssk);
        ssq = lanes_sum<LPC>(ssq);
        const float k_inv = rsqrtf(ssk + norm_eps), q_inv = rsqrtf(ssq + norm_eps) * q_scale;
        const float beta = sigmoid_f(bc);
        const float gdec = expf(-decay_rate * softplus_f(ac + bias));
        float ks = 0.f;
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            kc[r] *= k_inv;
            S[r] *= gdec;
            ks = fmaf(kc[r], S[r], ks);
        }
        ks = lanes_sum<LPC>(ks);
        const float u = beta * (vc - ks);
        float o = 0.f;
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            S[r] = fmaf(kc[r], u, S[r]);
            o = fmaf(qc[r], S[r], o);
        }
        o = lanes_sum<LPC>(o) * q_inv;
        if (sl == 0 && col_ok) out[((size_t)(t0 + i) * nh + h) * cols + col] = o;
        if (i + 1 < qlen) {
#pragma unroll
            for (int r = 0; r < RT; ++r) {
                kc[r] = kn[r];
                qc[r] = qn[r];
            }
            vc = vn; ac = an; bc = bn;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int r = 0; r < RT; ++r)
            if (r0 + r < rows) S_glob[(size_t)(r0 + r) * cols + col] = S[r];
    }
}

// Selective state space (Mamba-2).  Per token and head, with dt = softplus(dt_raw + dt_bias):
//   S <- exp(-exp(A_log) dt) S + dt B x^T;   y = S^T C + D x
// xbc [n, *]: x heads [nh, cols], then B [groups, rows], then C [groups, rows]; dt_raw [n, nh] at
// `dt` with its row stride.
template <typename T, int RT, int LPC>
__global__ void __launch_bounds__(REC_THREADS)
state_space_kernel(const T* __restrict__ xbc, long long xbc_stride, const T* __restrict__ dt, long long dt_stride,
                   const float* __restrict__ A_log, const float* __restrict__ dt_bias, const float* __restrict__ D,
                   float* __restrict__ state, long long slot_stride, const int* __restrict__ state_slots,
                   const int* __restrict__ cu_q, const int* __restrict__ positions, float* __restrict__ out, int nh,
                   int groups, int rows, int cols, int num_slots, int* __restrict__ status) {
    constexpr int CPB = REC_THREADS / LPC;
    const int s = blockIdx.z, h = blockIdx.y;
    const int col = blockIdx.x * CPB + threadIdx.x / LPC;
    const int sl = threadIdx.x % LPC;
    const int r0 = sl * RT;
    const int g = h / (nh / groups);
    const bool col_ok = col < cols;
    pdl_trigger();
    const int t0 = cu_q[s], qlen = cu_q[s + 1] - t0;
    if (qlen <= 0) return;
    const int slot = state_slots[s];
    if (slot < 0 || slot >= num_slots) {
        if (status) atomicExch(status, 3);
        return;
    }
    const float rate = expf(A_log[h]), bias = dt_bias[h], skip = D[h];
    const int b_off = nh * cols + g * rows, c_off = nh * cols + groups * rows + g * rows;
    float* S_glob = state + (size_t)slot * slot_stride + ((size_t)h * rows) * cols;
    const bool fresh = positions[t0] == 0;
    pdl_wait();
    float S[RT];
#pragma unroll
    for (int r = 0; r < RT; ++r)
        S[r] = (!fresh && col_ok && r0 + r < rows) ? S_glob[(size_t)(r0 + r) * cols + col] : 0.f;

    float Bc[RT], Cc[RT], xc, dc;
    auto fetch = [&](int t, float (&bb)[RT], float (&cc)[RT], float& xx, float& dd) {
        const T* row = xbc + (size_t)t * xbc_stride;
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            const bool ok = r0 + r < rows;
            bb[r] = ok ? to_f32(row[b_off + r0 + r]) : 0.f;
            cc[r] = ok ? to_f32(row[c_off + r0 + r]) : 0.f;
        }
        xx = col_ok ? to_f32(row[h * cols + col]) : 0.f;
        dd = to_f32(dt[(size_t)t * dt_stride + h]);
    };
    fetch(t0, Bc, Cc, xc, dc);
    for (int i = 0; i < qlen; ++i) {
        float Bn[RT], Cn[RT], xn = 0.f, dn = 0.f;
        if (i + 1 < qlen) fetch(t0 + i + 1, Bn, Cn, xn, dn);
        const float step = softplus_f(dc + bias);
        const float dec = expf(-rate * step);
        const float sx = step * xc;
        float y = 0.f;
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            S[r] = fmaf(dec, S[r], Bc[r] * sx);
            y = fmaf(Cc[r], S[r], y);
        }
        y = lanes_sum<LPC>(y);
        if (sl == 0 && col_ok) out[((size_t)(t0 + i) * nh + h) * cols + col] = fmaf(skip, xc, y);
        if (i + 1 < qlen) {
#pragma unroll
            for (int r = 0; r < RT; ++r) {
                Bc[r] = Bn[r];
                Cc[r] = Cn[r];
            }
            xc = xn; dc = dn;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int r = 0; r < RT; ++r)
            if (r0 + r < rows) S_glob[(size_t)(r0 + r) * cols + col] = S[r];
    }
}

// (RT, LPC) for a number of rows: the smallest product that holds them
#define REC_DISPATCH(ROWS, CALL)                                    \
    do {                                                            \
        if ((ROWS) <= 16) { CALL(4, 4); }                           \
        else if ((ROWS) <= 32) { CALL(8, 4); }                      \
        else if ((ROWS) <= 64) { CALL(8, 8); }                      \
        else if ((ROWS) <= 128) { CALL(16, 8); }                    \
        else { CALL(16, 16); }                                      \
    } while (0)

static inline int rec_lpc(int rows) { return rows <= 32 ? 4 : (rows <= 128 ? 8 : 16); }

VAPI_EXPORT int vapi_gated_delta(const void* qkv, long long qkv_stride, int q_off, int k_off, int v_off, const void* ab,
                                 long long ab_stride, int dtype, const float* A_log, const float* dt_bias, float* state,
                                 long long slot_stride, const int* state_slots, const int* cu_q, const int* positions,
                                 float* out, int num_seqs, int nh, int nkv, int rows, int cols, int num_slots,
                                 float norm_eps, int* status, cudaStream_t stream) {
    if (num_seqs <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || rows <= 0 || rows > 256 || cols <= 0)
        return fail(-1, "gated_delta: %d heads over %d, state %d x %d (rows up to 256)", nh, nkv, rows, cols);
    const int cpb = REC_THREADS / rec_lpc(rows);
    dim3 grid((cols + cpb - 1) / cpb, nh, num_seqs);
    cudaError_t e = cudaSuccess;
#define GD_CALL(RT, LPC)                                                                                                   \
    if (dtype == VAPI_F32)                                                                                                 \
        e = launch(gated_delta_kernel<float, RT, LPC>, grid, REC_THREADS, 0, stream, (const float*)qkv, qkv_stride, q_off, \
                   k_off, v_off, (const float*)ab, ab_stride, A_log, dt_bias, state, slot_stride, state_slots, cu_q,       \
                   positions, out, nh, nkv, rows, cols, num_slots, norm_eps, status);                                      \
    else                                                                                                                   \
        e = launch(gated_delta_kernel<__nv_bfloat16, RT, LPC>, grid, REC_THREADS, 0, stream, (const __nv_bfloat16*)qkv,    \
                   qkv_stride, q_off, k_off, v_off, (const __nv_bfloat16*)ab, ab_stride, A_log, dt_bias, state,            \
                   slot_stride, state_slots, cu_q, positions, out, nh, nkv, rows, cols, num_slots, norm_eps, status)
    if (dtype != VAPI_F32 && dtype != VAPI_BF16) return fail(-2, "gated_delta: unsupported dtype %d", dtype);
    REC_DISPATCH(rows, GD_CALL);
#undef GD_CALL
    return check_launch("gated_delta", e);
}

VAPI_EXPORT int vapi_state_space(const void* xbc, long long xbc_stride, const void* dt, long long dt_stride, int dtype,
                                 const float* A_log, const float* dt_bias, const float* D, float* state,
                                 long long slot_stride, const int* state_slots, const int* cu_q, const int* positions,
                                 float* out, int num_seqs, int nh, int groups, int rows, int cols, int num_slots,
                                 int* status, cudaStream_t stream) {
    if (num_seqs <= 0) return 0;
    if (nh <= 0 || groups <= 0 || nh % groups || rows <= 0 || rows > 256 || cols <= 0)
        return fail(-1, "state_space: %d heads over %d groups, state %d x %d (rows up to 256)", nh, groups, rows, cols);
    const int cpb = REC_THREADS / rec_lpc(rows);
    dim3 grid((cols + cpb - 1) / cpb, nh, num_seqs);
    cudaError_t e = cudaSuccess;
#define SS_CALL(RT, LPC)                                                                                                  \
    if (dtype == VAPI_F32)                                                                                                \
        e = launch(state_space_kernel<float, RT, LPC>, grid, REC_THREADS, 0, stream, (const float*)xbc, xbc_stride,       \
                   (const float*)dt, dt_stride, A_log, dt_bias, D, state, slot_stride, state_slots, cu_q, positions, out, \
                   nh, groups, rows, cols, num_slots, status);                                                            \
    else                                                                                                                  \
        e = launch(state_space_kernel<__nv_bfloat16, RT, LPC>, grid, REC_THREADS, 0, stream, (const __nv_bfloat16*)xbc,   \
                   xbc_stride, (const __nv_bfloat16*)dt, dt_stride, A_log, dt_bias, D, state, slot_stride, state_slots,   \
                   cu_q, positions, out, nh, groups, rows, cols, num_slots, status)
    if (dtype != VAPI_F32 && dtype != VAPI_BF16) return fail(-2, "state_space: unsupported dtype %d", dtype);
    REC_DISPATCH(rows, SS_CALL);
#undef SS_CALL
    return check_launch("state_space", e);
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
