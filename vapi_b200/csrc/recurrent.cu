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
                                        int channels, int L, int num_slots, int head_blocks, int* __restrict__ status, int act) {
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
            out[(size_t)(q0 + i) * channels + c] = from_f32<T>(act ? silu_f(acc) : acc);
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
    out[(size_t)t * channels + c] = from_f32<T>(act ? silu_f(acc) : acc);
}

// The (token, channel) part with 16-byte accesses: a thread takes VEC consecutive channels of one
// token (8 of bfloat16, 4 of float).  Rows of x, the taps and the output must be 16-byte aligned.
template <typename T> struct ConvVec;
template <> struct ConvVec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 f = *reinterpret_cast<const float4*>(p);
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct ConvVec<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 u = *reinterpret_cast<const uint4*>(p);
        const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
        unsigned w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 a = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<unsigned*>(&a);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

template <typename T>
__global__ void causal_conv_silu_vec_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ taps,
                                            const float* __restrict__ bias, const int* __restrict__ tok_seq,
                                            const int* __restrict__ cu_q, T* __restrict__ out, int n, int channels, int L, int act) {
    constexpr int VEC = ConvVec<T>::N;
    const int cv = channels / VEC;
    const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    pdl_trigger();
    if (item >= (long long)n * cv) {
        pdl_wait();
        return;
    }
    const int t = (int)(item / cv), c = (int)(item - (long long)t * cv) * VEC;
    const int i = t - cu_q[tok_seq[t]];
    if (i < L - 1) {                                        // a head token: the (sequence, channel) blocks' work
        pdl_wait();
        return;
    }
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; e += 4) {
        float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
        if (bias) b = *reinterpret_cast<const float4*>(bias + c + e);
        acc[e] = b.x; acc[e + 1] = b.y; acc[e + 2] = b.z; acc[e + 3] = b.w;
    }
    pdl_wait();
    for (int j = 0; j < L; ++j) {
        float xv[VEC];
        ConvVec<T>::load(x + (size_t)(t - (L - 1) + j) * x_stride + c, xv);
#pragma unroll
        for (int e = 0; e < VEC; e += 4) {
            const float4 w = *reinterpret_cast<const float4*>(taps + (size_t)j * channels + c + e);
            acc[e] = fmaf(w.x, xv[e], acc[e]);
            acc[e + 1] = fmaf(w.y, xv[e + 1], acc[e + 1]);
            acc[e + 2] = fmaf(w.z, xv[e + 2], acc[e + 2]);
            acc[e + 3] = fmaf(w.w, xv[e + 3], acc[e + 3]);
        }
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = act ? silu_f(acc[e]) : acc[e];
    ConvVec<T>::store(out + (size_t)t * channels + c, acc);
}

// act 1: SiLU behind the convolution; act 0: the convolution's sum as it is.
VAPI_EXPORT int vapi_causal_conv(const void* x, long long x_stride, int dtype, const float* taps, const float* bias,
                                 float* state, long long slot_stride, const int* state_slots, const int* tok_seq,
                                 const int* cu_q, const int* positions, void* out, int n, int num_seqs,
                                 int channels, int L, int num_slots, int max_q, int act, int* status, cudaStream_t stream) {
    if (n <= 0 || num_seqs <= 0) return 0;
    if (channels <= 0 || L < 1 || L > CONV_MAX_L) return fail(-1, "causal_conv_silu: %d channels, %d taps", channels, L);
    if (L > 1 && !state) return fail(-1, "causal_conv_silu: a convolution of %d taps needs a state", L);
    const int threads = 128;
    const int head_blocks = L > 1 ? (int)(((long long)num_seqs * channels + threads - 1) / threads) : 0;
    const int body_blocks = max_q > L - 1 ? (int)(((long long)n * channels + threads - 1) / threads) : 0;
    if (head_blocks + body_blocks == 0) return 0;
    cudaError_t e;
    const int vec = dtype == VAPI_BF16 ? 8 : 4;
    const size_t esz = dtype == VAPI_BF16 ? 2 : 4;
    if (body_blocks > 0 && (dtype == VAPI_F32 || dtype == VAPI_BF16) && channels % vec == 0 && x_stride % vec == 0 &&
        ((uintptr_t)x % 16) == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)taps % 16) == 0 && (!bias || ((uintptr_t)bias % 16) == 0) &&
        (x_stride * esz) % 16 == 0) {
        // the portions' first tokens and the states by (sequence, channel) threads, everything else 16 bytes at a time
        if (head_blocks > 0) {
            if (dtype == VAPI_F32)
                e = launch(causal_conv_silu_kernel<float>, head_blocks, threads, 0, stream, (const float*)x, x_stride, taps, bias, state,
                           slot_stride, state_slots, tok_seq, cu_q, positions, (float*)out, n, num_seqs, channels, L, num_slots,
                           head_blocks, status, act);
            else
                e = launch(causal_conv_silu_kernel<__nv_bfloat16>, head_blocks, threads, 0, stream, (const __nv_bfloat16*)x, x_stride,
                           taps, bias, state, slot_stride, state_slots, tok_seq, cu_q, positions, (__nv_bfloat16*)out, n, num_seqs,
                           channels, L, num_slots, head_blocks, status, act);
            const int rc = check_launch("causal_conv_silu", e);
            if (rc != 0) return rc;
        }
        const int vblocks = (int)(((long long)n * (channels / vec) + threads - 1) / threads);
        if (dtype == VAPI_F32)
            e = launch(causal_conv_silu_vec_kernel<float>, vblocks, threads, 0, stream, (const float*)x, x_stride, taps, bias, tok_seq,
                       cu_q, (float*)out, n, channels, L, act);
        else
            e = launch(causal_conv_silu_vec_kernel<__nv_bfloat16>, vblocks, threads, 0, stream, (const __nv_bfloat16*)x, x_stride, taps,
                       bias, tok_seq, cu_q, (__nv_bfloat16*)out, n, channels, L, act);
        return check_launch("causal_conv_silu", e);
    }
    if (dtype == VAPI_F32)
        e = launch(causal_conv_silu_kernel<float>, head_blocks + body_blocks, threads, 0, stream, (const float*)x, x_stride, taps,
                   bias, state, slot_stride, state_slots, tok_seq, cu_q, positions, (float*)out, n, num_seqs, channels, L,
                   num_slots, head_blocks, status, act);
    else if (dtype == VAPI_BF16)
        e = launch(causal_conv_silu_kernel<__nv_bfloat16>, head_blocks + body_blocks, threads, 0, stream, (const __nv_bfloat16*)x,
                   x_stride, taps, bias, state, slot_stride, state_slots, tok_seq, cu_q, positions, (__nv_bfloat16*)out, n,
                   num_seqs, channels, L, num_slots, head_blocks, status, act);
    else
        return fail(-2, "causal_conv_silu: unsupported dtype %d", dtype);
    return check_launch("causal_conv_silu", e);
}

VAPI_EXPORT int vapi_causal_conv_silu(const void* x, long long x_stride, int dtype, const float* taps, const float* bias,
                                      float* state, long long slot_stride, const int* state_slots, const int* tok_seq,
                                      const int* cu_q, const int* positions, void* out, int n, int num_seqs,
                                      int channels, int L, int num_slots, int max_q, int* status, cudaStream_t stream) {
    return vapi_causal_conv(x, x_stride, dtype, taps, bias, state, slot_stride, state_slots, tok_seq, cu_q, positions, out, n,
                            num_seqs, channels, L, num_slots, max_q, 1, status, stream);
}

// ---------------------------------------------------------------------------------------------
// The two recurrences share one decomposition.  The state of a head is a matrix S [rows, cols]
// (delta rule: key size x value size; state space: state size x head size).  A block owns one
// (sequence, head) and a slice of the columns and walks the sequence's tokens in order.  A column
// is shared by LPC neighbouring lanes, each holding RT consecutive rows of it in registers
// (RT * LPC >= rows); a sum over the rows ends with log2(LPC) shuffles.
//
// Tokens are taken REC_TC at a time: the block brings their row vectors (k and q, or B and C), its
// columns of v (or x) and their scalars into shared memory with coalesced loads, eight threads a
// token work out what the recurrence needs of them (unit-norm factors, the decay, the write strength,
// the dot product of the two row vectors), and then the REC_TC dependent steps read shared memory only.
// The loads of the next REC_TC tokens are in flight, in registers, while those steps run.  Both
// read-outs are rewritten over the state before the token's write, so that one round of shuffles
// serves a step:  o = S'^T q = (g S)^T q + (k.q) u  and  y = S'^T C = dec S^T C + step (B.C) x.
constexpr int REC_THREADS = 128;
constexpr int REC_TC = 16;

template <int LPC>
__device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
    for (int o = LPC >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// a row vector in shared memory: where a lane holds more than four rows, its rows are followed by four
// floats of padding, so that the LPC lanes of a column read 16-byte pieces that do not share banks
template <int RT>
__device__ __forceinline__ int rec_pad(int r) { return RT > 4 ? r + (r / RT) * 4 : r; }

// Stages the row vectors `a` and `b` [rows] and the block's columns `c` of REC_TC tokens.
template <typename T, int RT, int LPC>
struct RecStage {
    static constexpr int RP = RT * LPC;                       // rows, padded to what the lanes hold
    static constexpr int LANE = RT > 4 ? RT + 4 : RT;         // floats from one lane's rows to the next lane's
    static constexpr int RPP = LANE * LPC;                    // a row vector in shared memory
    static constexpr int CPB = REC_THREADS / LPC;
    static constexpr int NPT = REC_TC * RP / REC_THREADS;     // row elements per thread and vector
    static constexpr int VPT = (REC_TC * CPB + REC_THREADS - 1) / REC_THREADS;    // column elements per thread
    T ra[NPT], rb[NPT], rc[VPT];

    // requests the tokens first .. first + count - 1 (count <= REC_TC) into registers
    __device__ __forceinline__ void fetch(const T* __restrict__ src, long long stride, int a_off, int b_off, int c_off,
                                          int first, int count, int rows, int col0, int cols) {
#pragma unroll
        for (int e = 0; e < NPT; ++e) {
            const int idx = threadIdx.x + e * REC_THREADS;
            const int tt = idx / RP, r = idx - tt * RP;
            const bool ok = tt < count && r < rows;
            const T* row = src + (size_t)(first + tt) * stride;
            ra[e] = ok ? row[a_off + r] : from_f32<T>(0.f);
            rb[e] = ok ? row[b_off + r] : from_f32<T>(0.f);
        }
#pragma unroll
        for (int e = 0; e < VPT; ++e) {
            const int idx = threadIdx.x + e * REC_THREADS;
            const int tt = idx / CPB, c = idx - tt * CPB;
            const bool ok = idx < REC_TC * CPB && tt < count && col0 + c < cols;
            rc[e] = ok ? src[(size_t)(first + tt) * stride + c_off + col0 + c] : from_f32<T>(0.f);
        }
    }
    // writes what was requested to shared memory as float
    __device__ __forceinline__ void store(float* sa, float* sb, float* sc) const {
#pragma unroll
        for (int e = 0; e < NPT; ++e) {
            const int idx = threadIdx.x + e * REC_THREADS;
            const int tt = idx / RP, r = idx - tt * RP;
            sa[tt * RPP + rec_pad<RT>(r)] = to_f32(ra[e]);
            sb[tt * RPP + rec_pad<RT>(r)] = to_f32(rb[e]);
        }
#pragma unroll
        for (int e = 0; e < VPT; ++e)
            if (threadIdx.x + e * REC_THREADS < REC_TC * CPB) sc[threadIdx.x + e * REC_THREADS] = to_f32(rc[e]);
    }
};

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
    using Stage = RecStage<T, RT, LPC>;
    constexpr int CPB = Stage::CPB, RPP = Stage::RPP;
    __shared__ __align__(16) float sk[REC_TC * RPP], sq[REC_TC * RPP];
    __shared__ float sv[REC_TC * CPB], sg[REC_TC], sbeta[REC_TC], sqk[REC_TC], skinv[REC_TC], sqinv[REC_TC];
    const int s = blockIdx.z, h = blockIdx.y;
    const int col0 = blockIdx.x * CPB;
    const int col = col0 + threadIdx.x / LPC;
    const int sl = threadIdx.x % LPC;
    const int r0 = sl * RT;
    const int g = h / (nh / nkv);
    const bool col_ok = col < cols;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = cu_q[s], qlen = cu_q[s + 1] - t0;
    if (qlen <= 0) return;
    const int slot = state_slots[s];
    if (slot < 0 || slot >= num_slots) {
        if (threadIdx.x == 0 && status) atomicExch(status, 3);
        return;
    }
    const float decay_rate = expf(A_log[h]);
    const float bias = dt_bias[h];
    const float q_scale = rsqrtf((float)rows);
    float* S_glob = state + (size_t)slot * slot_stride + ((size_t)h * rows) * cols;
    const bool fresh = positions[t0] == 0;
    pdl_wait();
    float2 S2[RT / 2];                                      // this thread's rows of its column, two floats a register pair
#pragma unroll
    for (int r = 0; r < RT; r += 2) {
        S2[r / 2].x = (!fresh && col_ok && r0 + r < rows) ? S_glob[(size_t)(r0 + r) * cols + col] : 0.f;
        S2[r / 2].y = (!fresh && col_ok && r0 + r + 1 < rows) ? S_glob[(size_t)(r0 + r + 1) * cols + col] : 0.f;
    }

    Stage st;
    float a_raw = 0.f, b_raw = 0.f;
    auto fetch = [&](int first) {
        const int count = min(REC_TC, qlen - first);
        st.fetch(qkv, qkv_stride, k_off + g * rows, q_off + g * rows, v_off + h * cols, t0 + first, count, rows, col0, cols);
        if ((int)threadIdx.x < count) {
            a_raw = to_f32(ab[(size_t)(t0 + first + threadIdx.x) * ab_stride + h]);
            b_raw = to_f32(ab[(size_t)(t0 + first + threadIdx.x) * ab_stride + nh + h]);
        }
    };
    fetch(0);
    for (int first = 0; first < qlen; first += REC_TC) {
        const int count = min(REC_TC, qlen - first);
        __syncthreads();                                    // the steps of the last round have read shared memory
        st.store(sk, sq, sv);
        if ((int)threadIdx.x < count) {
            sg[threadIdx.x] = expf(-decay_rate * softplus_f(a_raw + bias));
            sbeta[threadIdx.x] = sigmoid_f(b_raw);
        }
        __syncthreads();
        if (first + REC_TC < qlen) fetch(first + REC_TC);   // in flight while these sixteen steps run
        // sums of squares and the dot product of k and q: eight threads a token, each an eighth of the rows
        {
            const int tt = threadIdx.x >> 3, part = threadIdx.x & 7;
            constexpr int PER = Stage::RP / 8;
            float ssk = 0.f, ssq = 0.f, dot = 0.f;
#pragma unroll
            for (int r = 0; r < (tt < count ? PER : 0); ++r) {
                const float kv = sk[tt * RPP + rec_pad<RT>(part * PER + r)], qv = sq[tt * RPP + rec_pad<RT>(part * PER + r)];
                ssk = fmaf(kv, kv, ssk);
                ssq = fmaf(qv, qv, ssq);
                dot = fmaf(kv, qv, dot);
            }
            ssk = lanes_sum<8>(ssk);
            ssq = lanes_sum<8>(ssq);
            dot = lanes_sum<8>(dot);
            if (part == 0) {
                const float k_inv = rsqrtf(ssk + norm_eps), q_inv = rsqrtf(ssq + norm_eps) * q_scale;
                skinv[tt] = k_inv;
                sqinv[tt] = q_inv;
                sqk[tt] = dot * k_inv * q_inv;
            }
        }
        __syncthreads();
#pragma unroll 2
        for (int tt = 0; tt < count; ++tt) {
            const float4* k4 = reinterpret_cast<const float4*>(sk + tt * RPP + sl * Stage::LANE);
            const float4* q4 = reinterpret_cast<const float4*>(sq + tt * RPP + sl * Stage::LANE);
            const float gdec = sg[tt];
            const float2 g2 = make_float2(gdec, gdec);
            float2 kc[RT / 2];
            float2 ks[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)}, qs[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
            for (int r4 = 0; r4 < RT / 4; ++r4) {            // (two floats an instruction: fma.rn.f32x2)
                const float4 kv = k4[r4], qv = q4[r4];
                kc[2 * r4] = make_float2(kv.x, kv.y);
                kc[2 * r4 + 1] = make_float2(kv.z, kv.w);
                S2[2 * r4] = __fmul2_rn(S2[2 * r4], g2);
                S2[2 * r4 + 1] = __fmul2_rn(S2[2 * r4 + 1], g2);
                ks[0] = __ffma2_rn(kc[2 * r4], S2[2 * r4], ks[0]);
                ks[1] = __ffma2_rn(kc[2 * r4 + 1], S2[2 * r4 + 1], ks[1]);
                qs[0] = __ffma2_rn(make_float2(qv.x, qv.y), S2[2 * r4], qs[0]);
                qs[1] = __ffma2_rn(make_float2(qv.z, qv.w), S2[2 * r4 + 1], qs[1]);
            }
            // (k and q stay as they came; their unit-norm factors multiply the sums)
            const float k_inv = skinv[tt];
            const float ksum = lanes_sum<LPC>((ks[0].x + ks[0].y) + (ks[1].x + ks[1].y)) * k_inv;
            const float qsum = lanes_sum<LPC>((qs[0].x + qs[0].y) + (qs[1].x + qs[1].y)) * sqinv[tt];
            const float u = sbeta[tt] * (sv[tt * CPB + threadIdx.x / LPC] - ksum);
            const float2 uk = make_float2(u * k_inv, u * k_inv);
#pragma unroll
            for (int r = 0; r < RT / 2; ++r) S2[r] = __ffma2_rn(kc[r], uk, S2[r]);
            if (sl == 0 && col_ok) out[((size_t)(t0 + first + tt) * nh + h) * cols + col] = fmaf(sqk[tt], u, qsum);
        }
    }
    pdl_trigger();                                          // (the next kernel is let go when the walk is over)
    if (col_ok) {
#pragma unroll
        for (int r = 0; r < RT; r += 2) {
            if (r0 + r < rows) S_glob[(size_t)(r0 + r) * cols + col] = S2[r / 2].x;
            if (r0 + r + 1 < rows) S_glob[(size_t)(r0 + r + 1) * cols + col] = S2[r / 2].y;
        }
    }
}

// Selective state space (Mamba-2).  Per token and head, with step = softplus(dt_raw + dt_bias):
//   S <- exp(-exp(A_log) step) S + step B x^T;   y = S^T C + D x
// xbc [n, *]: x heads [nh, cols], then B [groups, rows], then C [groups, rows]; dt_raw [n, nh] at
// `dt` with its row stride.
template <typename T, int RT, int LPC>
__global__ void __launch_bounds__(REC_THREADS)
state_space_kernel(const T* __restrict__ xbc, long long xbc_stride, const T* __restrict__ dt, long long dt_stride,
                   const float* __restrict__ A_log, const float* __restrict__ dt_bias, const float* __restrict__ D,
                   float* __restrict__ state, long long slot_stride, const int* __restrict__ state_slots,
                   const int* __restrict__ cu_q, const int* __restrict__ positions, float* __restrict__ out, int nh,
                   int groups, int rows, int cols, int num_slots, int* __restrict__ status) {
    using Stage = RecStage<T, RT, LPC>;
    constexpr int CPB = Stage::CPB, RPP = Stage::RPP;
    __shared__ __align__(16) float sB[REC_TC * RPP], sC[REC_TC * RPP];
    __shared__ float sx[REC_TC * CPB], sdec[REC_TC], sstep[REC_TC], sbc[REC_TC];
    const int s = blockIdx.z, h = blockIdx.y;
    const int col0 = blockIdx.x * CPB;
    const int col = col0 + threadIdx.x / LPC;
    const int sl = threadIdx.x % LPC;
    const int r0 = sl * RT;
    const int g = h / (nh / groups);
    const bool col_ok = col < cols;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = cu_q[s], qlen = cu_q[s + 1] - t0;
    if (qlen <= 0) return;
    const int slot = state_slots[s];
    if (slot < 0 || slot >= num_slots) {
        if (threadIdx.x == 0 && status) atomicExch(status, 3);
        return;
    }
    const float rate = expf(A_log[h]), bias = dt_bias[h], skip = D[h];
    const int b_off = nh * cols + g * rows, c_off = nh * cols + groups * rows + g * rows;
    float* S_glob = state + (size_t)slot * slot_stride + ((size_t)h * rows) * cols;
    const bool fresh = positions[t0] == 0;
    pdl_wait();
    float2 S2[RT / 2];
#pragma unroll
    for (int r = 0; r < RT; r += 2) {
        S2[r / 2].x = (!fresh && col_ok && r0 + r < rows) ? S_glob[(size_t)(r0 + r) * cols + col] : 0.f;
        S2[r / 2].y = (!fresh && col_ok && r0 + r + 1 < rows) ? S_glob[(size_t)(r0 + r + 1) * cols + col] : 0.f;
    }

    Stage st;
    float dt_raw = 0.f;
    auto fetch = [&](int first) {
        const int count = min(REC_TC, qlen - first);
        st.fetch(xbc, xbc_stride, b_off, c_off, h * cols, t0 + first, count, rows, col0, cols);
        if ((int)threadIdx.x < count) dt_raw = to_f32(dt[(size_t)(t0 + first + threadIdx.x) * dt_stride + h]);
    };
    fetch(0);
    for (int first = 0; first < qlen; first += REC_TC) {
        const int count = min(REC_TC, qlen - first);
        __syncthreads();
        st.store(sB, sC, sx);
        if ((int)threadIdx.x < count) {
            const float step = softplus_f(dt_raw + bias);
            sstep[threadIdx.x] = step;
            sdec[threadIdx.x] = expf(-rate * step);
        }
        __syncthreads();
        if (first + REC_TC < qlen) fetch(first + REC_TC);
        {
            const int tt = threadIdx.x >> 3, part = threadIdx.x & 7;
            constexpr int PER = Stage::RP / 8;
            float dot = 0.f;
#pragma unroll
            for (int r = 0; r < (tt < count ? PER : 0); ++r) dot = fmaf(sB[tt * RPP + rec_pad<RT>(part * PER + r)], sC[tt * RPP + rec_pad<RT>(part * PER + r)], dot);
            dot = lanes_sum<8>(dot);
            if (part == 0) sbc[tt] = dot;
        }
        __syncthreads();
#pragma unroll 2
        for (int tt = 0; tt < count; ++tt) {
            const float4* b4 = reinterpret_cast<const float4*>(sB + tt * RPP + sl * Stage::LANE);
            const float4* c4 = reinterpret_cast<const float4*>(sC + tt * RPP + sl * Stage::LANE);
            const float dec = sdec[tt];
            const float xv = sx[tt * CPB + threadIdx.x / LPC];
            const float sxv = sstep[tt] * xv;
            const float2 dec2 = make_float2(dec, dec), sx2 = make_float2(sxv, sxv);
            float2 cs[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
            for (int r4 = 0; r4 < RT / 4; ++r4) {            // (two floats an instruction: fma.rn.f32x2)
                const float4 bv = b4[r4], cv = c4[r4];
                cs[0] = __ffma2_rn(make_float2(cv.x, cv.y), S2[2 * r4], cs[0]);
                cs[1] = __ffma2_rn(make_float2(cv.z, cv.w), S2[2 * r4 + 1], cs[1]);
                S2[2 * r4] = __ffma2_rn(dec2, S2[2 * r4], __fmul2_rn(make_float2(bv.x, bv.y), sx2));
                S2[2 * r4 + 1] = __ffma2_rn(dec2, S2[2 * r4 + 1], __fmul2_rn(make_float2(bv.z, bv.w), sx2));
            }
            const float csum = lanes_sum<LPC>((cs[0].x + cs[0].y) + (cs[1].x + cs[1].y));       // C . S before the token's write
            if (sl == 0 && col_ok)
                out[((size_t)(t0 + first + tt) * nh + h) * cols + col] = fmaf(dec, csum, fmaf(sbc[tt], sxv, skip * xv));
        }
    }
    pdl_trigger();                                          // (the next kernel is let go when the walk is over)
    if (col_ok) {
#pragma unroll
        for (int r = 0; r < RT; r += 2) {
            if (r0 + r < rows) S_glob[(size_t)(r0 + r) * cols + col] = S2[r / 2].x;
            if (r0 + r + 1 < rows) S_glob[(size_t)(r0 + r + 1) * cols + col] = S2[r / 2].y;
        }
    }
}

// (RT, LPC) for a number of rows: the smallest product that holds them.  Few lanes per column mean many
// columns per block, and what a block does once per REC_TC tokens (staging, norms) is shared by all of
// them: measured at 128 rows and one sequence of 2,048 tokens, 16 lanes per column took 0.36 us a token
// against 0.31 us with 8 (and 1.0 against 1.6 TB/s of state traffic in decode steps of 64 sequences).
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
                                 float norm_eps, int max_q, int* status, cudaStream_t stream) {
    if (num_seqs <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv || rows <= 0 || rows > 256 || cols <= 0)
        return fail(-1, "gated_delta: %d heads over %d, state %d x %d (rows up to 256)", nh, nkv, rows, cols);
    const int cpb = REC_THREADS / rec_lpc(rows);
    dim3 grid((cols + cpb - 1) / cpb, nh, num_seqs);
    const bool early = max_q < REC_TC;                     // decode steps may start beside the kernel before; long walks may not
    cudaError_t e = cudaSuccess;
#define GD_CALL(RT, LPC)                                                                                                   \
    if (dtype == VAPI_F32)                                                                                                 \
        e = launch_if(early, gated_delta_kernel<float, RT, LPC>, grid, REC_THREADS, 0, stream, (const float*)qkv, qkv_stride, q_off, \
                   k_off, v_off, (const float*)ab, ab_stride, A_log, dt_bias, state, slot_stride, state_slots, cu_q,       \
                   positions, out, nh, nkv, rows, cols, num_slots, norm_eps, status);                                      \
    else                                                                                                                   \
        e = launch_if(early, gated_delta_kernel<__nv_bfloat16, RT, LPC>, grid, REC_THREADS, 0, stream, (const __nv_bfloat16*)qkv,    \
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
                                 int max_q, int* status, cudaStream_t stream) {
    if (num_seqs <= 0) return 0;
    if (nh <= 0 || groups <= 0 || nh % groups || rows <= 0 || rows > 256 || cols <= 0)
        return fail(-1, "state_space: %d heads over %d groups, state %d x %d (rows up to 256)", nh, groups, rows, cols);
    const int cpb = REC_THREADS / rec_lpc(rows);
    dim3 grid((cols + cpb - 1) / cpb, nh, num_seqs);
    const bool early = max_q < REC_TC;
    cudaError_t e = cudaSuccess;
#define SS_CALL(RT, LPC)                                                                                                  \
    if (dtype == VAPI_F32)                                                                                                \
        e = launch_if(early, state_space_kernel<float, RT, LPC>, grid, REC_THREADS, 0, stream, (const float*)xbc, xbc_stride,       \
                   (const float*)dt, dt_stride, A_log, dt_bias, D, state, slot_stride, state_slots, cu_q, positions, out, \
                   nh, groups, rows, cols, num_slots, status);                                                            \
    else                                                                                                                  \
        e = launch_if(early, state_space_kernel<__nv_bfloat16, RT, LPC>, grid, REC_THREADS, 0, stream, (const __nv_bfloat16*)xbc,   \
                   xbc_stride, (const __nv_bfloat16*)dt, dt_stride, A_log, dt_bias, D, state, slot_stride, state_slots,   \
                   cu_q, positions, out, nh, groups, rows, cols, num_slots, status)
    if (dtype != VAPI_F32 && dtype != VAPI_BF16) return fail(-2, "state_space: unsupported dtype %d", dtype);
    REC_DISPATCH(rows, SS_CALL);
#undef SS_CALL
    return check_launch("state_space", e);
}

VAPI_EXPORT const char* vapi_last_error() { return error_buffer(); }
