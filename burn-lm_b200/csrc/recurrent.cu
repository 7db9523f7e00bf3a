// Recurrent mixers over the packed tokens of a step: the short causal convolution with its carried inputs, the
// state-space scan (a scalar decay per head), the gated delta rule (a decay per key channel, an error-correcting
// write), and the group-wise RMS norm with a gate that follows either.  Everything here is fp32.
//
// What a sequence carries lives in a fixed-size block per cache slot, twice: a step that starts at position p reads
// copy (p & 1) and writes copy ((p + n) & 1) for its n new tokens.  A single-token step therefore never overwrites
// what it read, and running it again (a warm-up before a captured graph, a step enqueued ahead and then forgotten)
// gives the same result.  A step that starts at position 0 reads zeros whatever the block holds.
//
// A scan block owns (sequence, head, some value columns): 256 threads = columns x row groups; thread (col, rg) keeps rows
// rg, rg + RG, rg + 2 RG, ... of its column in registers.  A sum over rows is a thread's partial sum and then shuffles
// over the row groups (adjacent lanes): the same order whatever the step's size or batch.  RG = 8 (32 columns a block).
// More lanes a column were measured and left out.  RG = 32 (a warp a column, four times the warps): a 2,048-token scan of
// 64 heads x 128 rows x 64 lanes 0.97 against 0.86 ms, 64 single tokens 0.117 against 0.067 ms.  RG = 16: that scan 0.86
// against 0.79 ms (with the unrolled loop), the delta rule of 16 heads x 128 x 128 1.15 against 1.34 ms (its 64 blocks
// become 128), single tokens 0.089 against 0.072 and 0.069 against 0.050 ms: every block stages the same rows of B and C
// (or k, q and the decays) for fewer columns.  The state is stored as [head][row / RG][column][row % RG], which is the
// order in which a warp holds it, so RG belongs to a model's state and cannot change from step to step.  Fewer columns a
// block (16, in blocks of 128 threads, where a single sequence's 64 blocks would become 128) made the delta rule's prompt
// scan slower as well, 1.86 against 1.38 ms: the staging of a chunk is shared by fewer threads.
#include "common.cuh"

BLM_API const char* blm_recurrent_last_error() { return g_blm_error; }

constexpr int kMaxTaps = 16;
constexpr int kScanThreads = 256;
constexpr int kChunk = 32;         // tokens staged in shared memory at a time

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_r(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }

// ---------------------------------------------------------------------------------------------
// causal convolution per channel over time; act 1: then silu; act 2: the token's own input is added (y = x + conv(x))
//   x [N, x_stride] (channels at x_col0 ..), taps [C, K] (the last column is the current token's), bias [C] or null
//   carried inputs: hist [K - 1][C] per copy, hist[m] = the input at position start - (K - 1) + m
// ---------------------------------------------------------------------------------------------
__global__ void conv_kernel(const float* __restrict__ x, long long x_stride, int x_col0, int channels,
                            const float* __restrict__ taps, const float* __restrict__ bias, int K, int act,
                            float* __restrict__ out, long long out_stride, int out_col0,
                            const int* __restrict__ token_seq, const int* __restrict__ cu_seqlens,
                            const int* __restrict__ slot_of_seq, const int* __restrict__ start_pos,
                            float* __restrict__ state, long long slot_stride, long long copy_stride, long long hist_off,
                            int carry_here, __nv_bfloat16* __restrict__ out_bf, long long out_bf_stride) {
    const int n = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    float* o = out + (size_t)n * out_stride + out_col0 + c;
    const int seq = token_seq[n];
    if (seq < 0) {           // a row of no sequence
        *o = 0.f;
        if (out_bf) out_bf[(size_t)n * out_bf_stride + c] = __float2bfloat16(0.f);
        return;
    }
    const int i = n - cu_seqlens[seq];
    const int start = start_pos[seq];
    float* both = state + (size_t)slot_of_seq[seq] * slot_stride + hist_off;
    const float* hist = both + (size_t)(start & 1) * copy_stride;
    float acc = bias ? bias[c] : 0.f;
    for (int j = K - 1; j >= 0; --j) {          // the oldest input first
        const int back = i - j;                   // index among the step's rows of this sequence
        float v;
        if (back >= 0) v = x[(size_t)(n - j) * x_stride + x_col0 + c];
        else if (start + back < 0) v = 0.f;
        else v = hist[(size_t)(K - 1 + back) * channels + c];
        acc += taps[(size_t)c * K + (K - 1 - j)] * v;
    }
    if (act == 2) acc += x[(size_t)n * x_stride + x_col0 + c];      // the input itself joins what the taps give
    const float res = act == 1 ? silu_f(acc) : acc;
    *o = res;
    if (out_bf) out_bf[(size_t)n * out_bf_stride + c] = __float2bfloat16(res);
    if (carry_here) {        // every sequence brings one token: its thread also moves the carried inputs on, into the other copy
        float* fresh = both + (size_t)((start + 1) & 1) * copy_stride;
        for (int m = 0; m < K - 1; ++m) {
            const int p = start + 1 - (K - 1) + m;          // the position whose input goes to place m
            fresh[(size_t)m * channels + c] = p < 0 ? 0.f : (p == start ? x[(size_t)n * x_stride + x_col0 + c] : hist[(size_t)(m + 1) * channels + c]);
        }
    }
}

__global__ void conv_carry_kernel(const float* __restrict__ x, long long x_stride, int x_col0, int channels, int K,
                                  const int* __restrict__ cu_seqlens, const int* __restrict__ slot_of_seq,
                                  const int* __restrict__ start_pos, float* __restrict__ state, long long slot_stride,
                                  long long copy_stride, long long hist_off) {
    const int seq = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int first = cu_seqlens[seq];
    const int n_new = cu_seqlens[seq + 1] - first;
    if (n_new <= 0) return;      // an empty sequence (padding of a captured step)
    const int start = start_pos[seq];
    float* base = state + (size_t)slot_of_seq[seq] * slot_stride + hist_off;
    const float* old = base + (size_t)(start & 1) * copy_stride;
    float* fresh = base + (size_t)((start + n_new) & 1) * copy_stride;
    float keep[kMaxTaps];
#pragma unroll
    for (int m = 0; m < kMaxTaps - 1; ++m) {
        if (m < K - 1) {
            const int p = start + n_new - (K - 1) + m;      // the position whose input goes to place m
            float v;
            if (p < 0) v = 0.f;
            else if (p >= start) v = x[(size_t)(first + (p - start)) * x_stride + x_col0 + c];
            else v = old[(size_t)(K - 1 + (p - start)) * channels + c];
            keep[m] = v;
        }
    }
#pragma unroll
    for (int m = 0; m < kMaxTaps - 1; ++m)
        if (m < K - 1) fresh[(size_t)m * channels + c] = keep[m];
}

BLM_API int blm_causal_conv(const float* x, long long x_stride, int x_col0, int channels, const float* taps, const float* bias,
                            int K, int act, float* out, long long out_stride, int out_col0, const int* token_seq,
                            const int* cu_seqlens, const int* slot_of_seq, const int* start_pos, int n_tokens, int n_seqs,
                            float* state, long long slot_stride, long long copy_stride, long long hist_off,
                            int single_tokens, void* out_bf, long long out_bf_stride, cudaStream_t stream) {
    // out_bf (may be null): the result once more as bfloat16 [N, out_bf_stride], channel c in column c
    if (n_tokens == 0) return BLM_OK;
    BLM_REQUIRE(channels > 0 && K >= 1 && K <= kMaxTaps, "causal_conv: %d taps; this kernel takes 1 to %d", K, kMaxTaps);
    BLM_REQUIRE(n_tokens <= 65535 && n_seqs <= 65535, "causal_conv: a step of %d rows; this kernel takes 65,535", n_tokens);
    const int threads = 128;
    dim3 grid((channels + threads - 1) / threads, n_tokens);
    conv_kernel<<<grid, threads, 0, stream>>>(x, x_stride, x_col0, channels, taps, bias, K, act, out, out_stride, out_col0,
                                              token_seq, cu_seqlens, slot_of_seq, start_pos, state, slot_stride, copy_stride,
                                              hist_off, single_tokens && K > 1 ? 1 : 0, (__nv_bfloat16*)out_bf, out_bf_stride);
    int rc = blm_check_launch("causal_conv");
    if (rc != BLM_OK || K == 1 || single_tokens) return rc;
    dim3 grid2((channels + threads - 1) / threads, n_seqs);
    conv_carry_kernel<<<grid2, threads, 0, stream>>>(x, x_stride, x_col0, channels, K, cu_seqlens, slot_of_seq, start_pos, state,
                                                     slot_stride, copy_stride, hist_off);
    return blm_check_launch("causal_conv (carry)");
}

// ---------------------------------------------------------------------------------------------
// the scans
// ---------------------------------------------------------------------------------------------
struct ScanSeq {
    int first, n_new, start;
    const float* read;     // nullptr: the state is zero
    float* write;
};

__device__ __forceinline__ ScanSeq scan_seq(int seq, const int* cu_seqlens, const int* slot_of_seq, const int* start_pos,
                                            float* state, long long slot_stride, long long copy_stride, long long off) {
    ScanSeq s;
    s.first = cu_seqlens[seq];
    s.n_new = cu_seqlens[seq + 1] - s.first;
    s.start = start_pos[seq];
    float* base = state + (size_t)slot_of_seq[seq < 0 ? 0 : seq] * slot_stride + off;
    s.read = s.start > 0 ? base + (size_t)(s.start & 1) * copy_stride : nullptr;
    s.write = base + (size_t)((s.start + s.n_new) & 1) * copy_stride;
    return s;
}

template <int RG, typename V>
__device__ __forceinline__ V group_sum(V v) {       // over the row groups of a column (adjacent lanes)
#pragma unroll
    for (int o = 1; o < RG; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// State-space scan.  Per head h (group g = h / (heads / groups)), S [N x dv]:
//     S <- exp(-exp(A_log_h) dt) S + dt B x^T;   y = S^T C + D_h x,    dt = softplus(dt_raw + dt_bias_h)
// xbc [T, *]: x at x_col0 + h dv, B at b_col0 + g N, C at c_col0 + g N;  dt_raw [T, *] at dt_col0 + h.
// AT: the type the state is held and summed in inside a step.  float: the serving path.  double: the 32-bit path, where a
// head whose decay is close to 1 sums a thousand tokens into a state many times larger than its read-out (S^T C cancels),
// and float sums alone put 1e-5 of the row's largest value on it; the carried state is rounded to float either way.
template <int RN, int RG, typename AT>
__global__ void __launch_bounds__(kScanThreads)
    ssm_scan_kernel(const float* __restrict__ xbc, long long xbc_stride, int x_col0, int b_col0, int c_col0,
                    const float* __restrict__ dt_raw, long long dt_stride, int dt_col0, const float* __restrict__ dt_bias,
                    const float* __restrict__ A_log, const float* __restrict__ D, float* __restrict__ y, long long y_stride,
                    int heads, int groups, int N, int dv, const int* __restrict__ cu_seqlens, const int* __restrict__ slot_of_seq,
                    const int* __restrict__ start_pos, float* __restrict__ state, long long slot_stride, long long copy_stride,
                    long long state_off) {
    constexpr int NP = RN * RG, kCols = kScanThreads / RG, kRowGroups = RG;
    extern __shared__ __align__(16) float sm[];
    float* Bs = sm;                         // [kChunk][NP]
    float* Cs = Bs + kChunk * NP;           // [kChunk][NP]
    float* xs = Cs + kChunk * NP;           // [kChunk][kCols]
    AT* dts = reinterpret_cast<AT*>(xs + kChunk * kCols);       // [kChunk]  (an even number of floats lies before it)
    AT* decs = dts + kChunk;                                    // [kChunk]
    const int seq = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * kCols;
    const ScanSeq sq = scan_seq(seq, cu_seqlens, slot_of_seq, start_pos, state, slot_stride, copy_stride, state_off);
    if (sq.n_new <= 0) return;
    const int tid = threadIdx.x, col = tid / kRowGroups, rg = tid % kRowGroups;
    const int g = h / (heads / groups);
    const bool live = col0 + col < dv;
    const size_t head_off = (size_t)h * RN * dv * kRowGroups;
    AT s[RN];
#pragma unroll
    for (int r = 0; r < RN; ++r)
        s[r] = (sq.read && live) ? (AT)sq.read[head_off + ((size_t)r * dv + col0 + col) * kRowGroups + rg] : (AT)0;
    const float a = -expf(A_log[h]);
    const float bias = dt_bias[h], skip = D[h];
    for (int c0 = 0; c0 < sq.n_new; c0 += kChunk) {
        const int nt = min(kChunk, sq.n_new - c0);
        __syncthreads();
        for (int e = tid; e < nt * NP; e += blockDim.x) {
            const int t = e / NP, n = e % NP;
            const float* row = xbc + (size_t)(sq.first + c0 + t) * xbc_stride;
            Bs[e] = n < N ? row[b_col0 + g * N + n] : 0.f;
            Cs[e] = n < N ? row[c_col0 + g * N + n] : 0.f;
        }
        for (int e = tid; e < nt * kCols; e += blockDim.x) {
            const int t = e / kCols, p = e % kCols;
            xs[e] = col0 + p < dv ? xbc[(size_t)(sq.first + c0 + t) * xbc_stride + x_col0 + h * dv + col0 + p] : 0.f;
        }
        for (int t = tid; t < nt; t += blockDim.x) {
            const float dt = softplus_r(dt_raw[(size_t)(sq.first + c0 + t) * dt_stride + dt_col0 + h] + bias);
            dts[t] = (AT)dt;
            if (sizeof(AT) == 8) decs[t] = (AT)exp((double)a * (double)dt);
            else decs[t] = (AT)expf(a * dt);
        }
        __syncthreads();
        // (tokens unrolled: a token's shuffles and store wait for nothing the next token's multiply-adds need; the sum over
        // a thread's rows in four partial sums, so that no chain of dependent additions is longer than RN / 4)
#pragma unroll 4
        for (int t = 0; t < nt; ++t) {
            const AT dec = decs[t], dt = dts[t], xv = (AT)xs[t * kCols + col];
            const float* b = Bs + t * NP + rg;
            const float* c = Cs + t * NP + rg;
            AT part[4] = {0, 0, 0, 0};
#pragma unroll
            for (int r = 0; r < RN; ++r) {
                s[r] = dec * s[r] + (dt * (AT)b[r * kRowGroups]) * xv;
                part[r & 3] += s[r] * (AT)c[r * kRowGroups];
            }
            AT acc = (part[0] + part[1]) + (part[2] + part[3]);
            acc = group_sum<RG>(acc);
            if (rg == 0 && live) y[(size_t)(sq.first + c0 + t) * y_stride + h * dv + col0 + col] = (float)(acc + (AT)skip * xv);
        }
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < RN; ++r) sq.write[head_off + ((size_t)r * dv + col0 + col) * kRowGroups + rg] = (float)s[r];
    }
}

// Gated delta rule.  Per head h (query/key head c = h / (heads / qk_heads)), S [dk x dv]:
//     S <- g[:, None] S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
// with k, q made unit vectors (x / sqrt(sum x^2 + 1e-6)), q also times dk^(-1/2), beta = sigmoid(b_raw),
// g = exp(-exp(A_log_h) softplus(a_raw + dt_bias)) per head and key channel.
template <int RN, int RG>
__global__ void __launch_bounds__(kScanThreads)
    delta_scan_kernel(const float* __restrict__ q, long long q_stride, int q_col0, const float* __restrict__ k, long long k_stride,
                      int k_col0, const float* __restrict__ v, long long v_stride, int v_col0, const float* __restrict__ b_raw,
                      long long b_stride, int b_col0, const float* __restrict__ a_raw, long long a_stride, int a_col0,
                      const float* __restrict__ dt_bias, const float* __restrict__ A_log, float* __restrict__ o, long long o_stride,
                      int heads, int qk_heads, int dk, int dv, const int* __restrict__ cu_seqlens,
                      const int* __restrict__ slot_of_seq, const int* __restrict__ start_pos, float* __restrict__ state,
                      long long slot_stride, long long copy_stride, long long state_off) {
    constexpr int NP = RN * RG, kCols = kScanThreads / RG, kRowGroups = RG;
    extern __shared__ __align__(16) float sm[];
    float* ks = sm;                          // [kChunk][NP]
    float* qs = ks + kChunk * NP;            // [kChunk][NP]
    float* gs = qs + kChunk * NP;            // [kChunk][NP]
    float* vs = gs + kChunk * NP;            // [kChunk][kCols]
    float* betas = vs + kChunk * kCols;      // [kChunk]
    const int seq = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * kCols;
    const ScanSeq sq = scan_seq(seq, cu_seqlens, slot_of_seq, start_pos, state, slot_stride, copy_stride, state_off);
    if (sq.n_new <= 0) return;
    const int tid = threadIdx.x, col = tid / kRowGroups, rg = tid % kRowGroups;
    const int lane = tid & 31, warp = tid >> 5;
    const int c = h / (heads / qk_heads);
    const bool live = col0 + col < dv;
    const size_t head_off = (size_t)h * RN * dv * kRowGroups;
    float s[RN];
#pragma unroll
    for (int r = 0; r < RN; ++r)
        s[r] = (sq.read && live) ? sq.read[head_off + ((size_t)r * dv + col0 + col) * kRowGroups + rg] : 0.f;
    const float a = -expf(A_log[h]);
    const float q_scale = 1.0f / sqrtf((float)dk);
    for (int c0 = 0; c0 < sq.n_new; c0 += kChunk) {
        const int nt = min(kChunk, sq.n_new - c0);
        __syncthreads();
        for (int e = tid; e < nt * NP; e += blockDim.x) {
            const int t = e / NP, n = e % NP;
            const size_t row = (size_t)(sq.first + c0 + t);
            ks[e] = n < dk ? k[row * k_stride + k_col0 + c * dk + n] : 0.f;
            qs[e] = n < dk ? q[row * q_stride + q_col0 + c * dk + n] : 0.f;
            gs[e] = n < dk ? expf(a * softplus_r(a_raw[row * a_stride + a_col0 + h * dk + n] + dt_bias[h * dk + n])) : 1.f;
        }
        for (int e = tid; e < nt * kCols; e += blockDim.x) {
            const int t = e / kCols, p = e % kCols;
            vs[e] = col0 + p < dv ? v[(size_t)(sq.first + c0 + t) * v_stride + v_col0 + h * dv + col0 + p] : 0.f;
        }
        for (int t = tid; t < nt; t += blockDim.x)
            betas[t] = sigmoid_f(b_raw[(size_t)(sq.first + c0 + t) * b_stride + b_col0 + h]);
        __syncthreads();
        for (int t = warp; t < nt; t += blockDim.x / 32) {       // unit vectors: a warp per token
            float sk = 0.f, sqq = 0.f;
            for (int n = lane; n < NP; n += 32) {
                sk += ks[t * NP + n] * ks[t * NP + n];
                sqq += qs[t * NP + n] * qs[t * NP + n];
            }
            sk = warp_sum(sk);
            sqq = warp_sum(sqq);
            const float ik = 1.0f / sqrtf(sk + 1e-6f), iq = q_scale / sqrtf(sqq + 1e-6f);
            for (int n = lane; n < NP; n += 32) {
                ks[t * NP + n] *= ik;
                qs[t * NP + n] *= iq;
            }
        }
        __syncthreads();
#pragma unroll 2
        for (int t = 0; t < nt; ++t) {
            const float beta = betas[t], vv = vs[t * kCols + col];
            const float* kk = ks + t * NP + rg;
            const float* qq = qs + t * NP + rg;
            const float* gg = gs + t * NP + rg;
            float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r = 0; r < RN; ++r) {
                s[r] *= gg[r * kRowGroups];
                part[r & 3] += s[r] * kk[r * kRowGroups];
            }
            float acc = (part[0] + part[1]) + (part[2] + part[3]);
            acc = group_sum<RG>(acc);
            const float u = beta * (vv - acc);
            float outp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r = 0; r < RN; ++r) {
                s[r] += kk[r * kRowGroups] * u;
                outp[r & 3] += s[r] * qq[r * kRowGroups];
            }
            float out = (outp[0] + outp[1]) + (outp[2] + outp[3]);
            out = group_sum<RG>(out);
            if (rg == 0 && live) o[(size_t)(sq.first + c0 + t) * o_stride + h * dv + col0 + col] = out;
        }
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < RN; ++r) sq.write[head_off + ((size_t)r * dv + col0 + col) * kRowGroups + rg] = s[r];
    }
}


// ---------------------------------------------------------------------------------------------
// token shift: every one of S mixes of a token's input with the input of the token before it,
//     out[s][n] = x[n] + (x[n - 1] - x[n]) * mu[s]        (zeros before a sequence's first token)
// x float32 [N, x_stride]; mu float32 [S][C]; out [S][N][C].  The last input of every sequence is carried in `state`
// at hist_off, [C] per copy, as the convolution carries its inputs (it is the carried input of a convolution of two taps).
// ---------------------------------------------------------------------------------------------
template <typename TO>
__global__ void shift_mix_kernel(const float* __restrict__ x, long long x_stride, int channels, const float* __restrict__ mu, int S,
                                 TO* __restrict__ out, long long set_stride, const int* __restrict__ token_seq,
                                 const int* __restrict__ cu_seqlens, const int* __restrict__ slot_of_seq,
                                 const int* __restrict__ start_pos, float* __restrict__ state, long long slot_stride,
                                 long long copy_stride, long long hist_off, int carry_here) {
    const int n = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int seq = token_seq[n];
    if (seq < 0) {           // a row of no sequence
        for (int s = 0; s < S; ++s) out[(size_t)s * set_stride + (size_t)n * channels + c] = from_f32<TO>(0.f);
        return;
    }
    const int i = n - cu_seqlens[seq];
    const int start = start_pos[seq];
    float* both = state + (size_t)slot_of_seq[seq] * slot_stride + hist_off;
    const float cur = x[(size_t)n * x_stride + c];
    float prev;
    if (i > 0) prev = x[(size_t)(n - 1) * x_stride + c];
    else if (start == 0) prev = 0.f;
    else prev = both[(size_t)(start & 1) * copy_stride + c];
    const float diff = prev - cur;
    for (int s = 0; s < S; ++s)
        out[(size_t)s * set_stride + (size_t)n * channels + c] = from_f32<TO>(fmaf(diff, mu[(size_t)s * channels + c], cur));
    if (carry_here) both[(size_t)((start + 1) & 1) * copy_stride + c] = cur;
}

BLM_API int blm_shift_mix(const float* x, long long x_stride, int channels, const float* mu, int n_mixes, void* out, int out_dtype,
                          const int* token_seq, const int* cu_seqlens, const int* slot_of_seq, const int* start_pos, int n_tokens,
                          int n_seqs, float* state, long long slot_stride, long long copy_stride, long long hist_off,
                          int single_tokens, cudaStream_t stream) {
    if (n_tokens == 0) return BLM_OK;
    BLM_REQUIRE(channels > 0 && n_mixes > 0, "shift_mix: bad sizes");
    BLM_REQUIRE(n_tokens <= 65535 && n_seqs <= 65535, "shift_mix: a step of %d rows; this kernel takes 65,535", n_tokens);
    const int threads = 128;
    dim3 grid((channels + threads - 1) / threads, n_tokens);
    const long long set_stride = (long long)n_tokens * channels;
    if (out_dtype == BLM_F32)
        shift_mix_kernel<float><<<grid, threads, 0, stream>>>(x, x_stride, channels, mu, n_mixes, (float*)out, set_stride, token_seq,
                                                              cu_seqlens, slot_of_seq, start_pos, state, slot_stride, copy_stride,
                                                              hist_off, single_tokens ? 1 : 0);
    else if (out_dtype == BLM_BF16)
        shift_mix_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(x, x_stride, channels, mu, n_mixes, (__nv_bfloat16*)out, set_stride,
                                                                      token_seq, cu_seqlens, slot_of_seq, start_pos, state, slot_stride,
                                                                      copy_stride, hist_off, single_tokens ? 1 : 0);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "shift_mix: out dtype %d", out_dtype);
    int rc = blm_check_launch("shift_mix");
    if (rc != BLM_OK || single_tokens) return rc;
    dim3 grid2((channels + threads - 1) / threads, n_seqs);
    conv_carry_kernel<<<grid2, threads, 0, stream>>>(x, x_stride, 0, channels, 2, cu_seqlens, slot_of_seq, start_pos, state,
                                                     slot_stride, copy_stride, hist_off);
    return blm_check_launch("shift_mix (carry)");
}

// Linear attention with a decay per key channel.  Per head h, S [dk x dv]:
//     read first (a bonus u for the current token):   o = (S + diag(u) k v^T)^T q;   S <- diag(w) S + k v^T
//     read last:                                       S <- diag(w) S + k v^T;        o = S^T q
// What the raw inputs mean is the kind:
//     kDecayExpExp       w = exp(-exp(a + bias)),  q and k as they come            (bias [H dk]: the decays' base)
//     kDecayLowerBound   w = low + (1 - low) sigmoid(a + bias),  k = 1 - w,  q = silu(q)     (extra [H dk]: low)
// `extra` is the bonus u [H dk] when the state is read first.  AT as in the state-space scan: double holds the state and
// the sums over its rows in float64 inside a step (the 32-bit path).
constexpr int kDecayExpExp = 0, kDecayLowerBound = 1;

template <int RN, int RG, bool READ_FIRST, typename AT>
__global__ void __launch_bounds__(kScanThreads)
    decay_scan_kernel(const float* __restrict__ q, long long q_stride, int q_col0, const float* __restrict__ k, long long k_stride,
                      int k_col0, const float* __restrict__ v, long long v_stride, int v_col0, const float* __restrict__ a_raw,
                      long long a_stride, int a_col0, const float* __restrict__ bias, const float* __restrict__ extra,
                      float* __restrict__ o, long long o_stride, int heads, int dk, int dv, int kind,
                      const int* __restrict__ cu_seqlens, const int* __restrict__ slot_of_seq, const int* __restrict__ start_pos,
                      float* __restrict__ state, long long slot_stride, long long copy_stride, long long state_off) {
    constexpr int NP = RN * RG, kCols = kScanThreads / RG, kRowGroups = RG;
    extern __shared__ __align__(16) float sm[];
    float* ks = sm;                          // [kChunk][NP]
    float* qs = ks + kChunk * NP;            // [kChunk][NP]
    float* ws = qs + kChunk * NP;            // [kChunk][NP]
    float* vs = ws + kChunk * NP;            // [kChunk][kCols]
    const int seq = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * kCols;
    const ScanSeq sq = scan_seq(seq, cu_seqlens, slot_of_seq, start_pos, state, slot_stride, copy_stride, state_off);
    if (sq.n_new <= 0) return;
    const int tid = threadIdx.x, col = tid / kRowGroups, rg = tid % kRowGroups;
    const bool live = col0 + col < dv;
    const size_t head_off = (size_t)h * RN * dv * kRowGroups;
    AT s[RN];
    float ub[RN];
#pragma unroll
    for (int r = 0; r < RN; ++r) {
        s[r] = (sq.read && live) ? (AT)sq.read[head_off + ((size_t)r * dv + col0 + col) * kRowGroups + rg] : (AT)0;
        const int n = r * kRowGroups + rg;
        ub[r] = (READ_FIRST && extra && n < dk) ? extra[h * dk + n] : 0.f;
    }
    for (int c0 = 0; c0 < sq.n_new; c0 += kChunk) {
        const int nt = min(kChunk, sq.n_new - c0);
        __syncthreads();
        for (int e = tid; e < nt * NP; e += blockDim.x) {
            const int t = e / NP, n = e % NP;
            const size_t row = (size_t)(sq.first + c0 + t);
            float kk = 0.f, qq = 0.f, w = 1.f;
            if (n < dk) {
                const float a = a_raw[row * a_stride + a_col0 + h * dk + n] + bias[h * dk + n];
                qq = q[row * q_stride + q_col0 + h * dk + n];
                if (kind == kDecayExpExp) {
                    w = expf(-expf(a));
                    kk = k[row * k_stride + k_col0 + h * dk + n];
                } else {
                    const float low = extra[h * dk + n];
                    w = low + (1.0f - low) * sigmoid_f(a);
                    kk = 1.0f - w;
                    qq = silu_f(qq);
                }
            }
            ks[e] = kk;
            qs[e] = qq;
            ws[e] = w;
        }
        for (int e = tid; e < nt * kCols; e += blockDim.x) {
            const int t = e / kCols, p = e % kCols;
            vs[e] = col0 + p < dv ? v[(size_t)(sq.first + c0 + t) * v_stride + v_col0 + h * dv + col0 + p] : 0.f;
        }
        __syncthreads();
#pragma unroll 2
        for (int t = 0; t < nt; ++t) {
            const AT vv = (AT)vs[t * kCols + col];
            const float* kk = ks + t * NP + rg;
            const float* qq = qs + t * NP + rg;
            const float* ww = ws + t * NP + rg;
            AT part[4] = {0, 0, 0, 0};
#pragma unroll
            for (int r = 0; r < RN; ++r) {
                const AT kv = (AT)kk[r * kRowGroups] * vv;
                if (READ_FIRST) {
                    part[r & 3] += (s[r] + (AT)ub[r] * kv) * (AT)qq[r * kRowGroups];
                    s[r] = (AT)ww[r * kRowGroups] * s[r] + kv;
                } else {
                    s[r] = (AT)ww[r * kRowGroups] * s[r] + kv;
                    part[r & 3] += s[r] * (AT)qq[r * kRowGroups];
                }
            }
            AT acc = (part[0] + part[1]) + (part[2] + part[3]);
            acc = group_sum<RG>(acc);
            if (rg == 0 && live) o[(size_t)(sq.first + c0 + t) * o_stride + h * dv + col0 + col] = (float)acc;
        }
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < RN; ++r) sq.write[head_off + ((size_t)r * dv + col0 + col) * kRowGroups + rg] = (float)s[r];
    }
}

static int row_groups(int) { return 8; }
static int rows_per_thread(int n) {       // the smallest instance that holds n rows: row groups x RN
    for (int rn : {1, 2, 4, 8, 16, 32})
        if (rn * row_groups(n) >= n) return rn;
    return 0;
}

template <typename Kern>
static int allow_smem(Kern k, size_t smem, const char* what) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "%s: %s", what, cudaGetErrorString(e));
    }
    return BLM_OK;
}

BLM_API int blm_ssm_scan(const float* xbc, long long xbc_stride, int x_col0, int b_col0, int c_col0, const float* dt_raw,
                         long long dt_stride, int dt_col0, const float* dt_bias, const float* A_log, const float* D, float* y,
                         long long y_stride, int heads, int groups, int N, int dv, const int* cu_seqlens, const int* slot_of_seq,
                         const int* start_pos, int n_seqs, float* state, long long slot_stride, long long copy_stride,
                         long long state_off, int wide_sums, cudaStream_t stream) {
    if (n_seqs == 0) return BLM_OK;
    const int rn = rows_per_thread(N);
    BLM_REQUIRE(rn > 0, "ssm_scan: a state of %d rows; this kernel takes up to %d", N, 32 * 8);
    BLM_REQUIRE(heads > 0 && groups > 0 && heads % groups == 0 && dv > 0, "ssm_scan: bad head counts");
    BLM_REQUIRE(heads <= 65535 && dv <= 65535 * 8, "ssm_scan: too many heads");
    const int rg = row_groups(N), cols = kScanThreads / rg;
    dim3 grid(n_seqs, heads, (dv + cols - 1) / cols);
    const size_t smem = ((size_t)2 * kChunk * rn * rg + kChunk * cols) * sizeof(float) + 2 * kChunk * sizeof(double);
#define SSM_ARGS xbc, xbc_stride, x_col0, b_col0, c_col0, dt_raw, dt_stride, dt_col0, dt_bias, A_log, D, y, y_stride, heads, groups, N, dv, cu_seqlens, slot_of_seq, start_pos, state, slot_stride, copy_stride, state_off
#define BLM_SCAN(RN, RG)                                                                                 \
    if (rn == RN && rg == RG && wide_sums) {                                                             \
        int rc = allow_smem(ssm_scan_kernel<RN, RG, double>, smem, "ssm_scan_kernel");                   \
        if (rc != BLM_OK) return rc;                                                                     \
        ssm_scan_kernel<RN, RG, double><<<grid, kScanThreads, smem, stream>>>(SSM_ARGS);                 \
    }                                                                                                    \
    if (rn == RN && rg == RG && !wide_sums) {                                                            \
        int rc = allow_smem(ssm_scan_kernel<RN, RG, float>, smem, "ssm_scan_kernel");                    \
        if (rc != BLM_OK) return rc;                                                                     \
        ssm_scan_kernel<RN, RG, float><<<grid, kScanThreads, smem, stream>>>(xbc, xbc_stride, x_col0, b_col0, c_col0, dt_raw, dt_stride, dt_col0, dt_bias, A_log, D, y, y_stride, heads, groups, N, dv, cu_seqlens, slot_of_seq, start_pos, state, slot_stride, copy_stride, state_off); \
    }
    BLM_SCAN(1, 8) BLM_SCAN(2, 8) BLM_SCAN(4, 8) BLM_SCAN(8, 8) BLM_SCAN(16, 8) BLM_SCAN(32, 8)
#undef BLM_SCAN
#undef SSM_ARGS
    return blm_check_launch("ssm_scan");
}

BLM_API int blm_delta_scan(const float* q, long long q_stride, int q_col0, const float* k, long long k_stride, int k_col0,
                           const float* v, long long v_stride, int v_col0, const float* b_raw, long long b_stride, int b_col0,
                           const float* a_raw, long long a_stride, int a_col0, const float* dt_bias, const float* A_log, float* o,
                           long long o_stride, int heads, int qk_heads, int dk, int dv, const int* cu_seqlens,
                           const int* slot_of_seq, const int* start_pos, int n_seqs, float* state, long long slot_stride,
                           long long copy_stride, long long state_off, cudaStream_t stream) {
    if (n_seqs == 0) return BLM_OK;
    const int rn = rows_per_thread(dk);
    BLM_REQUIRE(rn > 0, "delta_scan: keys of %d lanes; this kernel takes up to %d", dk, 32 * 8);
    BLM_REQUIRE(heads > 0 && qk_heads > 0 && heads % qk_heads == 0 && dv > 0, "delta_scan: bad head counts");
    BLM_REQUIRE(heads <= 65535 && dv <= 65535 * 8, "delta_scan: too many heads");
    const int rg = row_groups(dk), cols = kScanThreads / rg;
    dim3 grid(n_seqs, heads, (dv + cols - 1) / cols);
    const size_t smem = ((size_t)3 * kChunk * rn * rg + kChunk * cols + 2 * kChunk) * sizeof(float);
#define BLM_SCAN(RN, RG)                                                                                 \
    if (rn == RN && rg == RG) {                                                                          \
        int rc = allow_smem(delta_scan_kernel<RN, RG>, smem, "delta_scan_kernel");                                   \
        if (rc != BLM_OK) return rc;                                                                     \
        delta_scan_kernel<RN, RG><<<grid, kScanThreads, smem, stream>>>(q, q_stride, q_col0, k, k_stride, k_col0, v, v_stride, v_col0, b_raw, b_stride, b_col0, a_raw, a_stride, a_col0, dt_bias, A_log, o, o_stride, heads, qk_heads, dk, dv, cu_seqlens, slot_of_seq, start_pos, state, slot_stride, copy_stride, state_off); \
    }
    BLM_SCAN(1, 8) BLM_SCAN(2, 8) BLM_SCAN(4, 8) BLM_SCAN(8, 8) BLM_SCAN(16, 8) BLM_SCAN(32, 8)
#undef BLM_SCAN
    return blm_check_launch("delta_scan");
}

BLM_API int blm_decay_scan(const float* q, long long q_stride, int q_col0, const float* k, long long k_stride, int k_col0,
                           const float* v, long long v_stride, int v_col0, const float* a_raw, long long a_stride, int a_col0,
                           const float* bias, const float* extra, float* o, long long o_stride, int heads, int dk, int dv, int kind,
                           int read_first, const int* cu_seqlens, const int* slot_of_seq, const int* start_pos, int n_seqs,
                           float* state, long long slot_stride, long long copy_stride, long long state_off, int wide_sums,
                           cudaStream_t stream) {
    if (n_seqs == 0) return BLM_OK;
    const int rn = rows_per_thread(dk);
    BLM_REQUIRE(rn > 0, "decay_scan: keys of %d lanes; this kernel takes up to %d", dk, 32 * 8);
    BLM_REQUIRE(heads > 0 && dv > 0 && heads <= 65535 && dv <= 65535 * 8, "decay_scan: bad head counts");
    BLM_REQUIRE(kind == kDecayExpExp || kind == kDecayLowerBound, "decay_scan: kind %d", kind);
    BLM_REQUIRE(kind != kDecayExpExp || k != nullptr, "decay_scan: this kind reads its keys");
    BLM_REQUIRE(kind != kDecayLowerBound || (extra != nullptr && !read_first), "decay_scan: a lower bound, and the state read last");
    const int rg = row_groups(dk), cols = kScanThreads / rg;
    dim3 grid(n_seqs, heads, (dv + cols - 1) / cols);
    const size_t smem = ((size_t)3 * kChunk * rn * rg + kChunk * cols) * sizeof(float);
#define DECAY_ARGS q, q_stride, q_col0, k, k_stride, k_col0, v, v_stride, v_col0, a_raw, a_stride, a_col0, bias, extra, o, o_stride, heads, dk, dv, kind, cu_seqlens, slot_of_seq, start_pos, state, slot_stride, copy_stride, state_off
#define BLM_ONE(RN, RG, FIRST, AT)                                                                       \
    {                                                                                                    \
        int rc = allow_smem(decay_scan_kernel<RN, RG, FIRST, AT>, smem, "decay_scan_kernel");            \
        if (rc != BLM_OK) return rc;                                                                     \
        decay_scan_kernel<RN, RG, FIRST, AT><<<grid, kScanThreads, smem, stream>>>(DECAY_ARGS);          \
    }
#define BLM_SCAN(RN, RG)                                                                                 \
    if (rn == RN && rg == RG) {                                                                          \
        if (read_first && wide_sums) BLM_ONE(RN, RG, true, double)                                       \
        else if (read_first) BLM_ONE(RN, RG, true, float)                                                \
        else if (wide_sums) BLM_ONE(RN, RG, false, double)                                               \
        else BLM_ONE(RN, RG, false, float)                                                               \
    }
    BLM_SCAN(1, 8) BLM_SCAN(2, 8) BLM_SCAN(4, 8) BLM_SCAN(8, 8) BLM_SCAN(16, 8) BLM_SCAN(32, 8)
#undef BLM_SCAN
#undef BLM_ONE
#undef DECAY_ARGS
    return blm_check_launch("decay_scan");
}

// ---------------------------------------------------------------------------------------------
// RMS norm over groups of a row's lanes, with a gate
//   mode 0 (gate first):  u = y silu(gate);  out = u / sqrt(mean_group(u^2) + eps) * w[lane % period]
//   mode 1 (gate last):   out = y / sqrt(mean_group(y^2) + eps) * w[lane % period] * sigmoid(gate)
//   mode 2 (silu last):   out = y / sqrt(mean_group(y^2) + eps) * w[lane % period] * silu(gate)
//   mode 3 (no gate):     out = y / sqrt(mean_group(y^2) + eps) * w[lane % period]            (gate may be null)
// A warp per (row, group).  Rows of no sequence hold zeros and give zeros.
// ---------------------------------------------------------------------------------------------
template <typename TA>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, long long y_stride, const float* __restrict__ gate,
                                        long long gate_stride, int gate_col0, const float* __restrict__ w, int period,
                                        int group, int n_groups, int mode, float eps, TA* __restrict__ out, long long out_stride) {
    const int n = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const float* yr = y + (size_t)n * y_stride;
    const float* gr = gate ? gate + (size_t)n * gate_stride + gate_col0 : nullptr;
    TA* orow = out + (size_t)n * out_stride;
    for (int g = warp; g < n_groups; g += n_warps) {
        const int lo = g * group;
        float ss = 0.f;
        for (int i = lane; i < group; i += 32) {
            float u = yr[lo + i];
            if (mode == 0) u *= silu_f(gr[lo + i]);
            ss += u * u;
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)group + eps);
        for (int i = lane; i < group; i += 32) {
            float u = yr[lo + i];
            const float gv = gr ? gr[lo + i] : 0.f;
            if (mode == 0) u = u * silu_f(gv) * inv * w[(lo + i) % period];
            else if (mode == 1) u = u * inv * w[(lo + i) % period] * sigmoid_f(gv);
            else if (mode == 2) u = u * inv * w[(lo + i) % period] * silu_f(gv);
            else u = u * inv * w[(lo + i) % period];
            orow[lo + i] = from_f32<TA>(u);
        }
    }
}

BLM_API int blm_gated_group_norm(const float* y, long long y_stride, const float* gate, long long gate_stride, int gate_col0,
                                 const float* w, int period, int group, int n_groups, int mode, float eps, void* out,
                                 int out_dtype, long long out_stride, int n, cudaStream_t stream) {
    if (n == 0) return BLM_OK;
    BLM_REQUIRE(group > 0 && n_groups > 0 && period > 0 && mode >= 0 && mode <= 3 && (gate != nullptr || mode == 3),
                "gated_group_norm: bad sizes or mode");
    const int threads = n_groups >= 8 ? 256 : 32 * n_groups;
    if (out_dtype == BLM_F32)
        gated_group_norm_kernel<float><<<n, threads, 0, stream>>>(y, y_stride, gate, gate_stride, gate_col0, w, period, group,
                                                                  n_groups, mode, eps, (float*)out, out_stride);
    else if (out_dtype == BLM_BF16)
        gated_group_norm_kernel<__nv_bfloat16><<<n, threads, 0, stream>>>(y, y_stride, gate, gate_stride, gate_col0, w, period,
                                                                          group, n_groups, mode, eps, (__nv_bfloat16*)out, out_stride);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "gated_group_norm: out dtype %d", out_dtype);
    return blm_check_launch("gated_group_norm");
}
