// Attention over a window of the latest keys plus the first keys of the sequence, with an optional sink in the
// softmax, keys and values of different sizes, and an optional gate per head.
//
//   visible(i, j) = j <= i and (i - j < window or j < keep_first)
//   p_j = exp(s_j) / (sink + sum_visible exp(s_j)),  s_j = scale q.k_j      (sink = 1: one more entry of score 0
//                                                                             that carries no value; 0: plain softmax)
//   out[n, h] = gate(n, h) * sum_j p_j v_j,  gate = sigmoid(g[n, h]) or 1
// Options of the scores (ScoreOpts): a number per query head that multiplies its scores, s_j = scale t_h q.k_j; a cap,
// s_j <- cap tanh(s_j / cap); and a score z_h of the sink other than 0, p_j = exp(s_j) / (exp(z_h) + sum exp(s_j)).
//
// The cache page of this family holds the keys [n_kv, page, dk] followed by the values [n_kv, page, dv].
// Scores, softmax and sums are fp32; q, keys and values are read in the cache's dtype.
#include "common.cuh"

BLM_API const char* blm_attention_sink_last_error() { return g_blm_error; }

// ---------------------------------------------------------------------------------------------
// After the fused projection [q | k | v | ...] (fp32 rows): the root mean square over the WHOLE q (all heads at
// once) and over the whole k, their weights, the blend of the values with an earlier layer's values of the same
// tokens, and the append of k and v to the token's place in the paged cache.
//   q_out[n, c] = q[c] / rms(q) * wq[c]            (wq == nullptr: q as it is)
//   k likewise; v <- (1 - lambda) v + lambda v_in[n] when v_in is given; v_out[n] = v when v_out is given
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void qk_norm_append_kernel(const float* __restrict__ proj, long long proj_stride, int q_cols, int k_cols, int v_cols,
                                      const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                                      const float* __restrict__ lambda_p, const float* __restrict__ v_in, float* __restrict__ v_out,
                                      T* __restrict__ q_out, T* __restrict__ pool, long long page_elems, int n_kv, int dk, int dv,
                                      int page_size, const int* __restrict__ token_seq, const int* __restrict__ token_pos,
                                      const int* __restrict__ slot_of_seq, const int* __restrict__ block_table, int table_stride) {
    __shared__ float red[33];
    const int n = blockIdx.x;
    const float* p = proj + (size_t)n * proj_stride;
    float rq = 1.f, rk = 1.f;
    if (wq != nullptr) {
        float sq = 0.f, sk = 0.f;
        for (int c = threadIdx.x; c < q_cols; c += blockDim.x) sq += p[c] * p[c];
        for (int c = threadIdx.x; c < k_cols; c += blockDim.x) sk += p[q_cols + c] * p[q_cols + c];
        sq = block_sum(sq, red);
        sk = block_sum(sk, red);
        rq = 1.0f / sqrtf(sq / (float)q_cols + eps);
        rk = 1.0f / sqrtf(sk / (float)k_cols + eps);
    }
    T* qo = q_out + (size_t)n * q_cols;
    for (int c = threadIdx.x; c < q_cols; c += blockDim.x) qo[c] = from_f32<T>(wq ? p[c] * rq * wq[c] : p[c]);
    const int seq = token_seq[n];
    T* kpage = nullptr;
    T* vpage = nullptr;
    int r = 0;
    if (seq >= 0) {
        const int pos = token_pos[n];
        const int page = block_table[(size_t)slot_of_seq[seq] * table_stride + pos / page_size];
        r = pos % page_size;
        kpage = pool + (size_t)page * page_elems;
        vpage = kpage + (size_t)n_kv * page_size * dk;
    }
    if (kpage != nullptr) {
        const float* k = p + q_cols;
        for (int c = threadIdx.x; c < k_cols; c += blockDim.x) {
            const int head = c / dk, d = c % dk;
            kpage[((size_t)head * page_size + r) * dk + d] = from_f32<T>(wk ? k[c] * rk * wk[c] : k[c]);
        }
    }
    const float lambda = v_in ? lambda_p[0] : 0.f;
    const float* v = p + q_cols + k_cols;
    for (int c = threadIdx.x; c < v_cols; c += blockDim.x) {
        float x = v[c];
        if (v_in) x = (1.0f - lambda) * x + lambda * v_in[(size_t)n * v_cols + c];
        if (v_out) v_out[(size_t)n * v_cols + c] = x;
        if (vpage != nullptr) {
            const int head = c / dv, d = c % dv;
            vpage[((size_t)head * page_size + r) * dv + d] = from_f32<T>(x);
        }
    }
}

BLM_API int blm_qk_norm_append(const float* proj, long long proj_stride, int n_tokens, int n_heads, int n_kv, int dk, int dv,
                               const float* wq, const float* wk, float eps, const float* lambda_p, const float* v_in, float* v_out,
                               void* q_out, void* pool, int dtype, long long page_elems, int page_size, const int* token_seq,
                               const int* token_pos, const int* slot_of_seq, const int* block_table, int table_stride,
                               cudaStream_t stream) {
    if (n_tokens == 0) return BLM_OK;
    BLM_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv > 0 && dk > 0 && dv > 0 && page_size > 0, "qk_norm_append: bad sizes");
    BLM_REQUIRE(page_elems == (long long)n_kv * page_size * (dk + dv), "qk_norm_append: a page holds n_kv * page * (dk + dv) elements");
    BLM_REQUIRE((wq == nullptr) == (wk == nullptr), "qk_norm_append: q and k are normed together or not at all");
    BLM_REQUIRE(v_in == nullptr || lambda_p != nullptr, "qk_norm_append: blending needs its weight");
    const int q_cols = n_heads * dk, k_cols = n_kv * dk, v_cols = n_kv * dv;
    if (dtype == BLM_F32)
        qk_norm_append_kernel<float><<<n_tokens, 256, 0, stream>>>(proj, proj_stride, q_cols, k_cols, v_cols, wq, wk, eps, lambda_p, v_in,
            v_out, (float*)q_out, (float*)pool, page_elems, n_kv, dk, dv, page_size, token_seq, token_pos, slot_of_seq, block_table,
            table_stride);
    else if (dtype == BLM_BF16)
        qk_norm_append_kernel<__nv_bfloat16><<<n_tokens, 256, 0, stream>>>(proj, proj_stride, q_cols, k_cols, v_cols, wq, wk, eps, lambda_p,
            v_in, v_out, (__nv_bfloat16*)q_out, (__nv_bfloat16*)pool, page_elems, n_kv, dk, dv, page_size, token_seq, token_pos,
            slot_of_seq, block_table, table_stride);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "qk_norm_append: dtype %d", dtype);
    return blm_check_launch("qk_norm_append");
}

// ---------------------------------------------------------------------------------------------
// The row kernel: one block per (query row, kv head, split of the keys), one warp per query head of the group (in
// turns when the group has more heads than the block has warps).  The visible keys of the row are walked in chunks
// of 32: the block stages a chunk's keys and values in shared memory (16-byte loads where the sizes allow), every
// lane of a warp scores one key, and the lanes then own the lanes of the output.  It serves single tokens, short
// portions, 32-bit prompts and every head size.  With several splits each block leaves (max, sum, unnormalised
// output) of its share of the keys and attention_sink_combine_kernel puts them together; the sink belongs to split 0.
// ---------------------------------------------------------------------------------------------
constexpr int kChunk = 32;
constexpr int kMaxVRegs = 16;     // value lanes per thread: dv <= 32 * kMaxVRegs

// `count` consecutive elements of a cache row (count a multiple of the vector width where `vec`) to fp32
template <typename T>
__device__ __forceinline__ void stage_row(float* dst, const T* src, int d0, bool vec);
template <>
__device__ __forceinline__ void stage_row<float>(float* dst, const float* src, int d0, bool vec) {
    if (vec) {
        const float4 a = *reinterpret_cast<const float4*>(src + d0), b = *reinterpret_cast<const float4*>(src + d0 + 4);
        dst[d0] = a.x; dst[d0 + 1] = a.y; dst[d0 + 2] = a.z; dst[d0 + 3] = a.w;
        dst[d0 + 4] = b.x; dst[d0 + 5] = b.y; dst[d0 + 6] = b.z; dst[d0 + 7] = b.w;
    } else {
        dst[d0] = src[d0];
    }
}
template <>
__device__ __forceinline__ void stage_row<__nv_bfloat16>(float* dst, const __nv_bfloat16* src, int d0, bool vec) {
    if (vec) {
        const uint4 raw = *reinterpret_cast<const uint4*>(src + d0);
        const __nv_bfloat162* pr = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(pr[e]);
            dst[d0 + 2 * e] = f.x;
            dst[d0 + 2 * e + 1] = f.y;
        }
    } else {
        dst[d0] = __bfloat162float(src[d0]);
    }
}

// ---------------------------------------------------------------------------------------------
// After the fused projection [q | k | v | ...] (fp32 rows), head by head:
//   q_h <- q_h / rms(q_h) * wq   (wq [dk], the same for every head; null: as it is), k_h likewise with wk;
//   the first rot_dims lanes of q_h and k_h turn by pos * freq[i]: lanes (2i, 2i + 1) when `halves` is 0, lanes
//   (i, i + rot_dims / 2) when it is 1; the other lanes pass;
//   v_h <- v_h / rms(v_h) when `value_norm` (no weight);
// q goes to q_out, k and v to the token's place in the paged cache.  rms(x) = sqrt(mean(x^2) + eps).  A warp a head;
// the angle, its sine and cosine in fp64, everything else fp32.
// ---------------------------------------------------------------------------------------------
// `turn`: (cosine, sine) of the token's angle for every pair of turning lanes, worked out once a token (all heads turn alike)
__device__ __forceinline__ float turned_lane(const float* src, const float* w, float inv, int j, int rot_dims, int halves,
                                             const float2* __restrict__ turn) {
    if (j >= rot_dims) return src[j] * inv * (w ? w[j] : 1.f);
    const int half = rot_dims >> 1;
    const int i = halves ? (j < half ? j : j - half) : (j >> 1);
    const int ia = halves ? i : 2 * i, ib = halves ? i + half : 2 * i + 1;
    const float a = src[ia] * inv * (w ? w[ia] : 1.f), b = src[ib] * inv * (w ? w[ib] : 1.f), cf = turn[i].x, sf = turn[i].y;
    return j == ib ? b * cf + a * sf : a * cf - b * sf;
}

template <typename T>
__global__ void head_norm_rope_append_kernel(const float* __restrict__ proj, long long proj_stride, int n_heads, int n_kv, int dk,
                                             int dv, const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                                             int value_norm, const double* __restrict__ freq, int rot_dims, int halves,
                                             T* __restrict__ q_out, T* __restrict__ pool, long long page_elems, int page_size,
                                             const int* __restrict__ token_seq, const int* __restrict__ token_pos,
                                             const int* __restrict__ slot_of_seq, const int* __restrict__ block_table,
                                             int table_stride) {
    extern __shared__ float2 turn[];                   // [rot_dims / 2]
    const int n = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const float* p = proj + (size_t)n * proj_stride;
    const int seq = token_seq[n];
    const bool real = seq >= 0;                        // a row of no sequence leaves zeros in q and reaches no cache
    const int pos = real ? token_pos[n] : 0;
    for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
        double sn, cs;
        sincos((double)pos * freq[i], &sn, &cs);
        turn[i] = make_float2((float)cs, (float)sn);
    }
    __syncthreads();
    T* kpage = nullptr;
    T* vpage = nullptr;
    int r = 0;
    if (real) {
        const int page = block_table[(size_t)slot_of_seq[seq] * table_stride + pos / page_size];
        r = pos % page_size;
        kpage = pool + (size_t)page * page_elems;
        vpage = kpage + (size_t)n_kv * page_size * dk;
    }
    const int n_vectors = n_heads + 2 * n_kv;          // the heads of q, then of k, then of v
    for (int item = warp; item < n_vectors; item += n_warps) {
        const bool is_q = item < n_heads, is_k = !is_q && item < n_heads + n_kv;
        const int head = is_q ? item : (is_k ? item - n_heads : item - n_heads - n_kv);
        const int width = (is_q || is_k) ? dk : dv;
        const float* src = p + (is_q ? (size_t)head * dk : (is_k ? (size_t)n_heads * dk + (size_t)head * dk
                                                                  : (size_t)(n_heads + n_kv) * dk + (size_t)head * dv));
        const float* w = is_q ? wq : (is_k ? wk : nullptr);
        float inv = 1.f;
        if (w != nullptr || (!is_q && !is_k && value_norm)) {
            float ss = 0.f;
            for (int d = lane; d < width; d += 32) ss += src[d] * src[d];
            ss = warp_sum(ss);
            inv = 1.0f / sqrtf(ss / (float)width + eps);
        }
        if (is_q) {
            T* dst = q_out + ((size_t)n * n_heads + head) * dk;
            for (int d = lane; d < dk; d += 32) dst[d] = from_f32<T>(real ? turned_lane(src, w, inv, d, rot_dims, halves, turn) : 0.f);
        } else if (is_k) {
            if (!real) continue;
            T* dst = kpage + ((size_t)head * page_size + r) * dk;
            for (int d = lane; d < dk; d += 32) dst[d] = from_f32<T>(turned_lane(src, w, inv, d, rot_dims, halves, turn));
        } else {
            if (!real) continue;
            T* dst = vpage + ((size_t)head * page_size + r) * dv;
            for (int d = lane; d < dv; d += 32) dst[d] = from_f32<T>(src[d] * inv);
        }
    }
}

BLM_API int blm_head_norm_rope_append(const float* proj, long long proj_stride, int n_tokens, int n_heads, int n_kv, int dk, int dv,
                                      const float* wq, const float* wk, float eps, int value_norm, const double* freq, int rot_dims,
                                      int halves, void* q_out, void* pool, int dtype, long long page_elems, int page_size,
                                      const int* token_seq, const int* token_pos, const int* slot_of_seq, const int* block_table,
                                      int table_stride, cudaStream_t stream) {
    if (n_tokens == 0) return BLM_OK;
    BLM_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv > 0 && dk > 0 && dv > 0 && page_size > 0, "head_norm_rope_append: bad sizes");
    BLM_REQUIRE(page_elems == (long long)n_kv * page_size * (dk + dv), "head_norm_rope_append: a page holds n_kv * page * (dk + dv) elements");
    BLM_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dk && (rot_dims == 0 || freq != nullptr),
                "head_norm_rope_append: %d turning lanes of %d", rot_dims, dk);
    const int vectors = n_heads + 2 * n_kv;
    const int threads = vectors >= 8 ? 256 : 32 * vectors;
#define BLM_HNRA(T)                                                                                                              \
    head_norm_rope_append_kernel<T><<<n_tokens, threads, (size_t)(rot_dims / 2 + 1) * sizeof(float2), stream>>>(proj, proj_stride, n_heads, n_kv, dk, dv, wq, wk, eps, value_norm, \
        freq, rot_dims, halves, (T*)q_out, (T*)pool, page_elems, page_size, token_seq, token_pos, slot_of_seq, block_table, table_stride)
    if (dtype == BLM_F32) BLM_HNRA(float);
    else if (dtype == BLM_BF16) BLM_HNRA(__nv_bfloat16);
    else return blm_fail(BLM_BAD_ARGUMENT, "head_norm_rope_append: dtype %d", dtype);
#undef BLM_HNRA
    return blm_check_launch("head_norm_rope_append");
}

// What a score goes through before the softmax, and what the sink weighs (all optional: null, null, 0).
struct ScoreOpts {
    const float* head_scale;     // [n_heads]: multiplies the head's scores beside `scale`
    const float* sink_logit;     // [n_heads]: the sink's score (null: 0); read only when the softmax has a sink
    float cap;                   // > 0: s <- cap tanh(s / cap)
};
__device__ __forceinline__ float capped(float s, float cap) { return cap > 0.f ? cap * tanhf(s / cap) : s; }
// The same for the tensor-core kernels, whose operands are bfloat16: tanh(x) = (1 - e) / (1 + e), e = exp(-2 |x|), by the
// special function unit (relative error about 1e-6, far below what the operands' rounding leaves in a score); the library's
// tanhf doubled those kernels' time.
__device__ __forceinline__ float capped_fast(float s, float cap, float inv_cap) {
    if (!(cap > 0.f)) return s;
    const float x = s * inv_cap;
    const float e = __expf(-2.0f * fabsf(x));
    return copysignf(cap * __fdividef(1.0f - e, 1.0f + e), x);
}

template <typename T>
__global__ void attention_sink_rows_kernel(const T* __restrict__ q, const T* __restrict__ pool, long long page_elems,
                                           const int* __restrict__ block_table, int table_stride, const int* __restrict__ token_seq,
                                           const int* __restrict__ token_pos, const int* __restrict__ slot_of_seq,
                                           const float* __restrict__ gate, long long gate_stride, T* __restrict__ out,
                                           float* __restrict__ partial, int n_heads, int n_kv, int dk, int dv, int page_size,
                                           int window, int keep_first, float scale, int sink, ScoreOpts so) {
    extern __shared__ float smem[];
    const int n = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z, n_splits = gridDim.z;
    const int group = n_heads / n_kv;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int kstride = dk + 1;                        // odd row length: the lanes of a warp read one column of 32 rows
    float* ks = smem;                                  // [kChunk][dk + 1]
    float* vs = ks + kChunk * kstride;                 // [kChunk][dv]
    float* qs = vs + kChunk * dv;                      // [n_warps][dk]
    const int seq = token_seq[n];
    T* orow = out + (size_t)n * n_heads * dv;
    if (seq < 0) {                                     // a row of no sequence: zeros, nothing read
        if (split == 0)
            for (int c = threadIdx.x; c < group * dv; c += blockDim.x) orow[(size_t)kvh * group * dv + c] = from_f32<T>(0.f);
        if (n_splits > 1)
            for (int c = threadIdx.x; c < group * (dv + 2); c += blockDim.x) {
                const int head = kvh * group + c / (dv + 2), e = c % (dv + 2);
                partial[(((size_t)n * n_heads + head) * n_splits + split) * (dv + 2) + e] = e == 0 ? -INFINITY : 0.f;
            }
        return;
    }
    const int pos = token_pos[n];
    const int* pages = block_table + (size_t)slot_of_seq[seq] * table_stride;
    const int lo = max(0, pos - window + 1);           // first key of the window
    const int n_first = min(keep_first, lo);           // kept first keys that lie before the window
    const int total = n_first + (pos - lo + 1);
    const int n_chunks = (total + kChunk - 1) / kChunk;
    const int per_split = (n_chunks + n_splits - 1) / n_splits;
    const int c_begin = split * per_split * kChunk, c_end = min(total, (split + 1) * per_split * kChunk);
    const bool kvec = (dk % 8) == 0, vvec = (dv % 8) == 0;       // rows start on 16-byte borders then (pages do always)
    const int kstep = kvec ? 8 : 1, vstep = vvec ? 8 : 1;
    const bool with_sink = sink && split == 0;
    for (int h0 = 0; h0 < group; h0 += n_warps) {
        const int head = kvh * group + h0 + warp;
        const bool active = h0 + warp < group;
        __syncthreads();                               // the chunk buffers and qs of the heads before are done with
        if (active)
            for (int d = lane; d < dk; d += 32) qs[warp * dk + d] = to_f32(q[((size_t)n * n_heads + head) * dk + d]);
        const float pre = scale * (active && so.head_scale ? so.head_scale[head] : 1.f);
        float m = with_sink ? (active && so.sink_logit ? so.sink_logit[head] : 0.f) : -INFINITY, l = with_sink ? 1.f : 0.f;
        float acc[kMaxVRegs];
#pragma unroll
        for (int i = 0; i < kMaxVRegs; ++i) acc[i] = 0.f;
        for (int c0 = c_begin; c0 < c_end; c0 += kChunk) {
            __syncthreads();
            for (int idx = threadIdx.x; idx < kChunk * (dk / kstep); idx += blockDim.x) {
                const int row = idx / (dk / kstep), d = (idx % (dk / kstep)) * kstep, i = c0 + row;
                if (i < c_end) {
                    const int j = i < n_first ? i : lo + (i - n_first);
                    const T* kpage = pool + (size_t)pages[j / page_size] * page_elems;
                    stage_row<T>(ks + row * kstride, kpage + ((size_t)kvh * page_size + j % page_size) * dk, d, kvec);
                }
            }
            for (int idx = threadIdx.x; idx < kChunk * (dv / vstep); idx += blockDim.x) {
                const int row = idx / (dv / vstep), d = (idx % (dv / vstep)) * vstep, i = c0 + row;
                if (i < c_end) {
                    const int j = i < n_first ? i : lo + (i - n_first);
                    const T* vpage = pool + (size_t)pages[j / page_size] * page_elems + (size_t)n_kv * page_size * dk;
                    stage_row<T>(vs + row * dv, vpage + ((size_t)kvh * page_size + j % page_size) * dv, d, vvec);
                }
            }
            __syncthreads();
            if (active) {
                const bool mine = c0 + lane < c_end;
                float s = -INFINITY;
                if (mine) {
                    float dot = 0.f;
                    const float* kr = ks + lane * kstride;
                    const float* qr = qs + warp * dk;
                    for (int d = 0; d < dk; ++d) dot = fmaf(qr[d], kr[d], dot);
                    s = capped(dot * pre, so.cap);
                }
                const float m_new = fmaxf(m, warp_max(s));      // finite: the chunk has a key
                const float p = mine ? expf(s - m_new) : 0.f;
                const float corr = expf(m - m_new);             // m = -inf only before the first chunk
                l = l * corr + warp_sum(p);
                m = m_new;
#pragma unroll
                for (int i = 0; i < kMaxVRegs; ++i) acc[i] *= corr;
                const int rows = min(kChunk, c_end - c0);
                for (int j = 0; j < rows; ++j) {
                    const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
                    for (int i = 0; i < kMaxVRegs; ++i) {
                        const int d = lane + 32 * i;
                        if (d < dv) acc[i] = fmaf(pj, vs[j * dv + d], acc[i]);
                    }
                }
            }
        }
        if (active && n_splits > 1) {
            float* part = partial + (((size_t)n * n_heads + head) * n_splits + split) * (dv + 2);
            if (lane == 0) {
                part[0] = m;
                part[1] = l;
            }
#pragma unroll
            for (int i = 0; i < kMaxVRegs; ++i) {
                const int d = lane + 32 * i;
                if (d < dv) part[2 + d] = acc[i];
            }
        } else if (active) {
            float g = 1.f;
            if (gate != nullptr) g = 1.0f / (1.0f + expf(-gate[(size_t)n * gate_stride + head]));
            const float inv = l > 0.f ? g / l : 0.f;
#pragma unroll
            for (int i = 0; i < kMaxVRegs; ++i) {
                const int d = lane + 32 * i;
                if (d < dv) orow[(size_t)head * dv + d] = from_f32<T>(acc[i] * inv);
            }
        }
    }
}

// out[n, head] = gate * sum_z acc_z e^(m_z - M) / sum_z l_z e^(m_z - M),  M = max_z m_z: one warp per (row, head)
template <typename T>
__global__ void attention_sink_combine_kernel(const float* __restrict__ partial, const float* __restrict__ gate, long long gate_stride,
                                              T* __restrict__ out, int n_rows, int n_heads, int dv, int n_splits) {
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= n_rows * n_heads) return;
    const int n = item / n_heads, head = item % n_heads;
    const float* part = partial + (size_t)item * n_splits * (dv + 2);
    float big = -INFINITY;
    for (int z = 0; z < n_splits; ++z) big = fmaxf(big, part[(size_t)z * (dv + 2)]);
    float l = 0.f;
    for (int z = 0; z < n_splits; ++z) {
        const float mz = part[(size_t)z * (dv + 2)];
        if (mz > -INFINITY) l += part[(size_t)z * (dv + 2) + 1] * expf(mz - big);
    }
    float g = 1.f;
    if (gate != nullptr) g = 1.0f / (1.0f + expf(-gate[(size_t)n * gate_stride + head]));
    const float inv = l > 0.f ? g / l : 0.f;
    for (int d = lane; d < dv; d += 32) {
        float a = 0.f;
        for (int z = 0; z < n_splits; ++z) {
            const float mz = part[(size_t)z * (dv + 2)];
            if (mz > -INFINITY) a += part[(size_t)z * (dv + 2) + 2 + d] * expf(mz - big);
        }
        out[((size_t)n * n_heads + head) * dv + d] = from_f32<T>(a * inv);
    }
}

template <typename T>
static int launch_rows(const void* q, const void* pool, long long page_elems, const int* block_table, int table_stride,
                       const int* token_seq, const int* token_pos, const int* slot_of_seq, const float* gate, long long gate_stride,
                       void* out, float* partial, int n_splits, int n_tokens, int n_heads, int n_kv, int dk, int dv, int page_size,
                       int window, int keep_first, float scale, int sink, ScoreOpts so, cudaStream_t stream) {
    const int group = n_heads / n_kv;
    const int warps = group < 8 ? group : 8;
    const size_t smem = ((size_t)kChunk * (dk + 1) + (size_t)kChunk * dv + (size_t)warps * dk) * sizeof(float);
    if (smem > 48 * 1024) {
        BLM_REQUIRE(smem <= 200 * 1024, "attention_sink: heads of %d and %d lanes need %zu bytes of shared memory", dk, dv, smem);
        cudaError_t e = cudaFuncSetAttribute(attention_sink_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "attention_sink: %s", cudaGetErrorString(e));
    }
    attention_sink_rows_kernel<T><<<dim3(n_tokens, n_kv, n_splits), warps * 32, smem, stream>>>(
        (const T*)q, (const T*)pool, page_elems, block_table, table_stride, token_seq, token_pos, slot_of_seq, gate, gate_stride,
        (T*)out, partial, n_heads, n_kv, dk, dv, page_size, window, keep_first, scale, sink, so);
    if (n_splits > 1) {
        const int items = n_tokens * n_heads;
        attention_sink_combine_kernel<T><<<(items + 3) / 4, 128, 0, stream>>>(partial, gate, gate_stride, (T*)out, n_tokens, n_heads, dv,
                                                                              n_splits);
    }
    return blm_check_launch("attention_sink");
}

// ---------------------------------------------------------------------------------------------
// The tensor-core kernels (bfloat16, mma.sync m16n8k16 with fp32 sums, operands fetched with ldmatrix).  Keys and
// values come a cache page (64 positions) at a time through cp.async into two buffers in turn, so that the next page
// is on its way while this one is worked on: first the pages of the kept first tokens that lie wholly before the
// window, then the pages from the window's start to the last query.  Keys that a query must not see are masked by
// position; the values of keys beyond the last query are staged as zeros, so that what a page's unused rows hold
// never meets the sums.  NV: value lanes in tiles of 8 (dv <= 8 NV); dk and dv are multiples of 8.
//
// Prompt kernel: a block of four warps per (64 query rows of one sequence, query head); a warp owns 16 query rows, so
// a row's softmax stays inside a quad of lanes.
// Decode kernel: a block per (token, kv head, split of the pages); the rows of the tile are the query heads of the
// group (up to 16), and each warp takes 16 of a page's 64 keys with a running softmax of its own; the four are put
// together at the end.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned smem_at(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// four 8x8 tiles of 16-bit elements from shared memory (`a`: a 32-bit shared address, see smem_at): lanes 8i .. 8i + 7
// give the addresses of the rows of tile i; a lane receives, of
// every tile, the elements (lane / 4, 2 (lane % 4)) and the next (transposed: (2 (lane % 4), lane / 4) and the one below)
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], unsigned a) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], unsigned a) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
// 16 bytes from global to shared memory without passing registers; `valid` false: zeros instead (nothing is read)
__device__ __forceinline__ void cp_async16(__nv_bfloat16* dst, const __nv_bfloat16* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait_all_but() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
#ifndef BLM_PROMPT_STAGES
#define BLM_PROMPT_STAGES 2
#endif
constexpr int kPromptStages = BLM_PROMPT_STAGES;       // pages of the prompt kernel in shared memory: one worked on, the others on their way

// 2^x by the special function unit (the scores are in units of log 2; -inf gives 0)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// zeros where no copy will write: rows [row_begin, n_rows) of a staged operand wholly, and lanes [used, stride) of the others
__device__ __forceinline__ void zero_unwritten(__nv_bfloat16* buf, int n_rows, int stride, int row_begin, int used) {
    const int vec = stride / 8;
    for (int idx = threadIdx.x; idx < n_rows * vec; idx += blockDim.x) {
        const int r = idx / vec, c = (idx % vec) * 8;
        if (r >= row_begin || c >= used) *reinterpret_cast<uint4*>(buf + r * stride + c) = make_uint4(0u, 0u, 0u, 0u);
    }
}

constexpr int kTileQ = 64, kTileK = 64;

// The pages a query tile walks: `kept` pages from the sequence's start, then pages wp0 .. wp1.
struct PageWalk {
    int kept, wp0, n_tiles;
    __device__ __forceinline__ PageWalk(int p_first, int p_last, int window, int keep_first) {
        const int lo = max(0, p_first - window + 1);
        wp0 = lo / kTileK;
        kept = min((keep_first + kTileK - 1) / kTileK, wp0);
        n_tiles = kept + (p_last / kTileK - wp0 + 1);
    }
    __device__ __forceinline__ int page(int it) const { return it < kept ? it : wp0 + (it - kept); }
};

// How one thread of a block walks a [rows][vec] grid of 16-byte groups that the block's threads share out in turn:
// where it starts and how far a step of blockDim groups takes it (worked out once: the walk itself divides nothing).
struct GroupWalk {
    int r, c, dr, dc, vec;
    __device__ __forceinline__ GroupWalk(int vec_) : vec(vec_) {
        r = threadIdx.x / vec_;
        c = threadIdx.x % vec_;
        dr = blockDim.x / vec_;
        dc = blockDim.x % vec_;
    }
};

// one page's keys and values of one kv head into a buffer pair (every thread of the block takes its share)
__device__ __forceinline__ void stage_page(__nv_bfloat16* kbuf, __nv_bfloat16* vbuf, const __nv_bfloat16* page, int n_kv, int kvh, int dk,
                                           int dv, int qstride, int vstride, int first_pos, int p_last, const GroupWalk& kw,
                                           const GroupWalk& vw) {
    const __nv_bfloat16* kpage = page + (size_t)kvh * kTileK * dk;
    const __nv_bfloat16* vpage = page + (size_t)n_kv * kTileK * dk + (size_t)kvh * kTileK * dv;
    for (int r = kw.r, c = kw.c; r < kTileK;) {
        cp_async16(kbuf + r * qstride + c * 8, kpage + r * dk + c * 8, true);
        r += kw.dr;
        c += kw.dc;
        if (c >= kw.vec) {
            c -= kw.vec;
            ++r;
        }
    }
    for (int r = vw.r, c = vw.c; r < kTileK;) {
        cp_async16(vbuf + r * vstride + c * 8, vpage + r * dv + c * 8, first_pos + r <= p_last);
        r += vw.dr;
        c += vw.dc;
        if (c >= vw.vec) {
            c -= vw.vec;
            ++r;
        }
    }
}

template <int NV, int HB>
__global__ void __launch_bounds__(128 * HB) attention_sink_prompt_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pool, long long page_elems,
    const int* __restrict__ block_table, int table_stride, const int* __restrict__ cu_seqlens, const int* __restrict__ start_pos,
    const int* __restrict__ slot_of_seq, int n_seqs, int n_tokens, const float* __restrict__ gate, long long gate_stride,
    __nv_bfloat16* __restrict__ out, int n_heads, int n_kv, int dk, int dv, int window, int keep_first, float scale, int sink,
    ScoreOpts so) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int found[3];
    const int tid = threadIdx.x, lane = tid & 31, warp = (tid >> 5) & 3, hb = tid >> 7;     // hb: which of the block's heads
    const int dkp = (dk + 15) & ~15;                   // the reduction runs in steps of 16 lanes; the rest is zeros
    const int qstride = dkp + 8;                       // rows 16 bytes apart modulo 128: ldmatrix reads eight of them at once
    constexpr int vstride = 8 * NV + 8;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [HB][64][qstride]
    __nv_bfloat16* Kb = Qs + HB * kTileQ * qstride;                      // kPromptStages x [64][qstride]
    __nv_bfloat16* Vb = Kb + kPromptStages * kTileK * qstride;           // kPromptStages x [64][vstride]
    const int head = blockIdx.y * HB + hb;             // the block's heads share a kv head (HB divides the group)
    if (tid == 0) {
        int t = blockIdx.x;
        found[0] = -1;
        for (int s = 0; s < n_seqs; ++s) {
            const int len = cu_seqlens[s + 1] - cu_seqlens[s];
            const int tiles = (len + kTileQ - 1) / kTileQ;
            if (t < tiles) {
                found[0] = s;
                found[1] = t * kTileQ;
                found[2] = len;
                break;
            }
            t -= tiles;
        }
    }
    __syncthreads();
    if (found[0] < 0) {
        // a block without a tile: the rows after the last sequence (padding up to a captured step's size) get zeros
        const int end = cu_seqlens[n_seqs];
        for (int idx = tid & 127; idx < (n_tokens - end) * dv; idx += 128)
            out[((size_t)(end + idx / dv) * n_heads + head) * dv + idx % dv] = __float2bfloat16_rn(0.f);
        return;
    }
    const int seq = found[0], t0 = found[1], len = found[2];
    const int kvh = head / (n_heads / n_kv);
    const int row0 = cu_seqlens[seq] + t0;             // the tile's first token row
    const int rows = min(kTileQ, len - t0);
    const int p0 = start_pos[seq] + t0;                // its position
    const int p_last = p0 + rows - 1;
    const int* pages = block_table + (size_t)slot_of_seq[seq] * table_stride;
    // zeros where no copy writes: rows of no query, lanes beyond dk and dv (the copies take whole groups of 8 lanes)
#pragma unroll
    for (int i = 0; i < HB; ++i) zero_unwritten(Qs + i * kTileQ * qstride, kTileQ, qstride, rows, dk);
    zero_unwritten(Kb, kPromptStages * kTileK, qstride, kPromptStages * kTileK, dk);
    zero_unwritten(Vb, kPromptStages * kTileK, vstride, kPromptStages * kTileK, dv);
    const PageWalk walk(p0, p_last, window, keep_first);
    for (int idx = tid & 127; idx < rows * (dk / 8); idx += 128) {       // every group of four warps brings its head's queries
        const int r = idx / (dk / 8), c = (idx % (dk / 8)) * 8;
        cp_async16(Qs + (hb * kTileQ + r) * qstride + c, q + ((size_t)(row0 + r) * n_heads + head) * dk + c, true);
    }
    const GroupWalk kw(dk / 8), vw(dv / 8);
    auto fetch = [&](int it) {                         // page `it` of the walk into its place in the ring
        const int pg = walk.page(it), b = it % kPromptStages;
        stage_page(Kb + b * kTileK * qstride, Vb + b * kTileK * vstride, pool + (size_t)pages[pg] * page_elems, n_kv, kvh, dk, dv, qstride,
                   vstride, pg * kTileK, p_last, kw, vw);
    };
#pragma unroll
    for (int ahead = 0; ahead < kPromptStages - 1; ++ahead) {
        if (ahead < walk.n_tiles) fetch(ahead);
        cp_async_commit();
    }
    const int quad = lane >> 2, pair = (lane & 3) * 2;
    const int lrow = lane & 7, lmat = lane >> 3;
    const int pr0 = p0 + warp * 16 + quad, pr1 = pr0 + 8;        // positions of this thread's two rows
    // scores in units of log 2: the exponentials are exp2.  A cap (or a head's multiplier that is not positive, under which
    // the largest raw score is not the largest score) is applied to the raw scores first, which are then in natural units.
    const float pre = scale * (so.head_scale ? so.head_scale[head] : 1.f);
    const bool shaped = so.cap > 0.f || !(pre > 0.f);
    const float scale2 = (shaped ? 1.f : pre) * 1.4426950408889634f;
    const float inv_cap = so.cap > 0.f ? 1.0f / so.cap : 0.f;
    float m[2], l[2], o[NV][4];
    m[0] = m[1] = sink ? (so.sink_logit ? so.sink_logit[head] * 1.4426950408889634f : 0.f) : -INFINITY;
    l[0] = l[1] = sink ? 0.25f : 0.f;                  // a quad's four lanes add up to the sink's one
#pragma unroll
    for (int j = 0; j < NV; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    const unsigned qa = smem_at(Qs + (hb * kTileQ + warp * 16 + lrow + (lmat & 1) * 8) * qstride + (lmat >> 1) * 8);
    const unsigned kb0 = smem_at(Kb + (lrow + (lmat >> 1) * 8) * qstride + (lmat & 1) * 8);
    const unsigned vb0 = smem_at(Vb + (lrow + (lmat & 1) * 8) * vstride + (lmat >> 1) * 8);
    const unsigned kstep = 16 * qstride * 2;           // bytes from 16 keys to the next 16
    for (int it = 0; it < walk.n_tiles; ++it) {
        const int buf = it % kPromptStages;
        if (it + kPromptStages - 1 < walk.n_tiles) fetch(it + kPromptStages - 1);      // into the buffer the page before has left
        cp_async_commit();
        cp_async_wait_all_but<kPromptStages - 1>();    // this page (and the queries) have landed; the others may be on their way
        __syncthreads();
        const int pg = walk.page(it);
        const unsigned kb = kb0 + buf * kTileK * qstride * 2, vb = vb0 + buf * kTileK * vstride * 2;
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        for (int kk = 0; kk < dkp; kk += 16) {
            uint32_t a[4], b[4];
            ldsm_x4(a, qa + kk * 2);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                ldsm_x4(b, kb + jj * kstep + kk * 2);
                mma_bf16(s[2 * jj], a, b[0], b[1]);
                mma_bf16(s[2 * jj + 1], a, b[2], b[3]);
            }
        }
        if (shaped) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = capped_fast(s[j][e] * pre, so.cap, inv_cap);
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
        // every row of this warp sees every key of the page when the page lies behind the warp's first row and inside
        // the window of its last (or among the kept first tokens): then nothing is masked (most pages of a long window)
        const int w_first = p0 + warp * 16, w_last = w_first + 15, key0 = pg * kTileK;
        if (key0 + kTileK - 1 <= w_first && (w_last - key0 < window || key0 + kTileK <= keep_first)) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
                mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + 8 * j + pair + (e & 1);
                    const int pr = e < 2 ? pr0 : pr1;
                    const bool sees = key <= pr && (pr - key < window || key < keep_first);
                    const float v = sees ? s[j][e] : -INFINITY;
                    s[j][e] = v;
                    if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
                }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        // the running maxima are kept in units of log 2 (scale2 > 0: the largest raw score is the largest score)
        const float mn0 = fmaxf(m[0], mx0 * scale2), mn1 = fmaxf(m[1], mx1 * scale2);
        const float use0 = mn0 == -INFINITY ? 0.f : mn0, use1 = mn1 == -INFINITY ? 0.f : mn1;    // a row that has seen no key yet
        const float corr0 = fast_exp2(m[0] - use0), corr1 = fast_exp2(m[1] - use1);
        m[0] = mn0;
        m[1] = mn1;
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            s[j][0] = fast_exp2(fmaf(s[j][0], scale2, -use0)); s[j][1] = fast_exp2(fmaf(s[j][1], scale2, -use0));
            s[j][2] = fast_exp2(fmaf(s[j][2], scale2, -use1)); s[j][3] = fast_exp2(fmaf(s[j][3], scale2, -use1));
            sum0 += s[j][0] + s[j][1];
            sum1 += s[j][2] + s[j][3];
        }
        l[0] = l[0] * corr0 + sum0;
        l[1] = l[1] * corr1 + sum1;
        if (corr0 != 1.f || corr1 != 1.f) {            // once the maxima have settled there is nothing to rescale
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                o[j][0] *= corr0; o[j][1] *= corr0;
                o[j][2] *= corr1; o[j][3] *= corr1;
            }
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {               // 16 keys a step: two of the score tiles make one operand
            uint32_t a[4], b[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]); a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]); a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int jj = 0; jj < NV / 2; ++jj) {
                ldsm_x4_trans(b, vb + (16 * kk * vstride + 16 * jj) * 2);
                mma_bf16(o[2 * jj], a, b[0], b[1]);
                mma_bf16(o[2 * jj + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();                               // the buffer may be filled again
    }
    l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
    l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
    l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
    l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
    const int r0 = warp * 16 + quad, r1 = r0 + 8;
    float inv0 = 0.f, inv1 = 0.f;
    if (r0 < rows) {
        const float g = gate ? 1.0f / (1.0f + expf(-gate[(size_t)(row0 + r0) * gate_stride + head])) : 1.f;
        inv0 = l[0] > 0.f ? g / l[0] : 0.f;
    }
    if (r1 < rows) {
        const float g = gate ? 1.0f / (1.0f + expf(-gate[(size_t)(row0 + r1) * gate_stride + head])) : 1.f;
        inv1 = l[1] > 0.f ? g / l[1] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int d = 8 * j + pair;
        if (d < dv) {
            if (r0 < rows)
                *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r0) * n_heads + head) * dv + d) = pack_bf16(o[j][0] * inv0, o[j][1] * inv0);
            if (r1 < rows)
                *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r1) * n_heads + head) * dv + d) = pack_bf16(o[j][2] * inv1, o[j][3] * inv1);
        }
    }
}

template <int NV, int HB>
static int launch_prompt(const void* q, const void* pool, long long page_elems, const int* block_table, int table_stride,
                         const int* cu_seqlens, const int* start_pos, const int* slot_of_seq, int n_seqs, const float* gate,
                         long long gate_stride, void* out, int n_tokens, int n_heads, int n_kv, int dk, int dv, int window,
                         int keep_first, float scale, int sink, ScoreOpts so, cudaStream_t stream) {
    const int dkp = (dk + 15) & ~15;
    const size_t smem = ((size_t)(HB + kPromptStages) * kTileQ * (dkp + 8) + (size_t)kPromptStages * kTileK * (8 * NV + 8)) * sizeof(__nv_bfloat16);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attention_sink_prompt_kernel<NV, HB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "attention_sink: %s", cudaGetErrorString(e));
    }
    cudaFuncSetAttribute(attention_sink_prompt_kernel<NV, HB>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    const unsigned tiles = (unsigned)((n_tokens + kTileQ - 1) / kTileQ + n_seqs);     // every sequence may end in a tile that is not full
    attention_sink_prompt_kernel<NV, HB><<<dim3(tiles, n_heads / HB), 128 * HB, smem, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)pool, page_elems, block_table, table_stride, cu_seqlens, start_pos, slot_of_seq,
        n_seqs, n_tokens, gate, gate_stride, (__nv_bfloat16*)out, n_heads, n_kv, dk, dv, window, keep_first, scale, sink, so);
    return blm_check_launch("attention_sink (prompt)");
}

// kDecodeStages pages in shared memory, one worked on and the others on their way.  Measured with 64 sequences of
// 1,088 tokens on 8 kv heads: heads of 64 lanes 45 us with two stages (five blocks to a multiprocessor), 60 with three,
// 61 with four; heads of 128 lanes 84, 79 and 121 us.

template <int NV, int kDecodeStages>
__global__ void __launch_bounds__(128) attention_sink_decode_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pool, long long page_elems,
    const int* __restrict__ block_table, int table_stride, const int* __restrict__ token_seq, const int* __restrict__ token_pos,
    const int* __restrict__ slot_of_seq, const float* __restrict__ gate, long long gate_stride, __nv_bfloat16* __restrict__ out,
    float* __restrict__ partial, int n_heads, int n_kv, int dk, int dv, int window, int keep_first, float scale, int sink,
    ScoreOpts so) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z, n_splits = gridDim.z;
    const int group = n_heads / n_kv;                  // <= 16: the rows of the tile
    const int dkp = (dk + 15) & ~15;
    const int qstride = dkp + 8;
    constexpr int vstride = 8 * NV + 8;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [16][qstride]
    __nv_bfloat16* Kb = Qs + 16 * qstride;                               // kDecodeStages x [64][qstride]
    __nv_bfloat16* Vb = Kb + kDecodeStages * kTileK * qstride;           // kDecodeStages x [64][vstride]
    const int seq = token_seq[n];
    const int head0 = kvh * group;
    if (seq < 0) {                                     // a row of no sequence: zeros, nothing read
        if (split == 0)
            for (int c = tid; c < group * dv; c += 128) out[((size_t)n * n_heads + head0) * dv + c] = __float2bfloat16_rn(0.f);
        if (n_splits > 1)
            for (int c = tid; c < group * (dv + 2); c += 128) {
                const int head = head0 + c / (dv + 2), e = c % (dv + 2);
                partial[(((size_t)n * n_heads + head) * n_splits + split) * (dv + 2) + e] = e == 0 ? -INFINITY : 0.f;
            }
        return;
    }
    const int pos = token_pos[n];
    const int* pages = block_table + (size_t)slot_of_seq[seq] * table_stride;
    zero_unwritten(Qs, 16, qstride, group, dk);
    zero_unwritten(Kb, kDecodeStages * kTileK, qstride, kDecodeStages * kTileK, dk);
    zero_unwritten(Vb, kDecodeStages * kTileK, vstride, kDecodeStages * kTileK, dv);
    const PageWalk walk(pos, pos, window, keep_first);
    const int per_split = (walk.n_tiles + n_splits - 1) / n_splits;
    const int it_begin = split * per_split, it_end = min(walk.n_tiles, it_begin + per_split);
    for (int idx = tid; idx < group * (dk / 8); idx += 128) {
        const int r = idx / (dk / 8), c = (idx % (dk / 8)) * 8;
        cp_async16(Qs + r * qstride + c, q + ((size_t)n * n_heads + head0 + r) * dk + c, true);
    }
    const GroupWalk kw(dk / 8), vw(dv / 8);
    auto fetch = [&](int it) {                         // page `it` of the walk into its place in the ring
        const int pg = walk.page(it), b = (it - it_begin) % kDecodeStages;
        stage_page(Kb + b * kTileK * qstride, Vb + b * kTileK * vstride, pool + (size_t)pages[pg] * page_elems, n_kv, kvh, dk, dv, qstride,
                   vstride, pg * kTileK, pos, kw, vw);
    };
#pragma unroll
    for (int ahead = 0; ahead < kDecodeStages - 1; ++ahead) {
        if (it_begin + ahead < it_end) fetch(it_begin + ahead);
        cp_async_commit();
    }
    const int quad = lane >> 2, pair = (lane & 3) * 2;
    const int lrow = lane & 7, lmat = lane >> 3;
    const bool with_sink = sink && split == 0 && warp == 0;      // the sink is counted once
    const float log2e = 1.4426950408889634f;                     // scores in units of log 2: the exponentials are exp2
    float m[2], l[2], o[NV][4], pre[2];
    const float inv_cap = so.cap > 0.f ? 1.0f / so.cap : 0.f;
#pragma unroll
    for (int half = 0; half < 2; ++half) {                       // this thread's two rows are two heads of the group
        const int r = quad + 8 * half;
        pre[half] = scale * (so.head_scale && r < group ? so.head_scale[head0 + r] : 1.f);
        m[half] = with_sink ? (so.sink_logit && r < group ? so.sink_logit[head0 + r] * log2e : 0.f) : -INFINITY;
        l[half] = with_sink ? 0.25f : 0.f;
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    const unsigned qa = smem_at(Qs + (lrow + (lmat & 1) * 8) * qstride + (lmat >> 1) * 8);
    // this warp's 16 keys of a page
    const unsigned kb0 = smem_at(Kb + (16 * warp + lrow + (lmat >> 1) * 8) * qstride + (lmat & 1) * 8);
    const unsigned vb0 = smem_at(Vb + (16 * warp + lrow + (lmat & 1) * 8) * vstride + (lmat >> 1) * 8);
    for (int it = it_begin; it < it_end; ++it) {
        const int buf = (it - it_begin) % kDecodeStages;
        if (it + kDecodeStages - 1 < it_end) fetch(it + kDecodeStages - 1);      // into the buffer the page before this one has left
        cp_async_commit();
        cp_async_wait_all_but<kDecodeStages - 1>();    // this page (and the queries) have landed; the others may be on their way
        __syncthreads();
        const int pg = walk.page(it);
        const unsigned kb = kb0 + buf * kTileK * qstride * 2, vb = vb0 + buf * kTileK * vstride * 2;
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
        for (int kk = 0; kk < dkp; kk += 16) {
            uint32_t a[4], b[4];
            ldsm_x4(a, qa + kk * 2);
            ldsm_x4(b, kb + kk * 2);
            mma_bf16(s[0], a, b[0], b[1]);
            mma_bf16(s[1], a, b[2], b[3]);
        }
        // every row (head) sees the same keys
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = pg * kTileK + 16 * warp + 8 * j + pair + (e & 1);
                const bool sees = key <= pos && (pos - key < window || key < keep_first);
                s[j][e] = sees ? capped_fast(s[j][e] * pre[e >> 1], so.cap, inv_cap) * log2e : -INFINITY;
            }
        float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        float mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
        const float use0 = mn0 == -INFINITY ? 0.f : mn0, use1 = mn1 == -INFINITY ? 0.f : mn1;
        const float corr0 = fast_exp2(m[0] - use0), corr1 = fast_exp2(m[1] - use1);
        m[0] = mn0;
        m[1] = mn1;
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            s[j][0] = fast_exp2(s[j][0] - use0); s[j][1] = fast_exp2(s[j][1] - use0);
            s[j][2] = fast_exp2(s[j][2] - use1); s[j][3] = fast_exp2(s[j][3] - use1);
            sum0 += s[j][0] + s[j][1];
            sum1 += s[j][2] + s[j][3];
        }
        l[0] = l[0] * corr0 + sum0;
        l[1] = l[1] * corr1 + sum1;
        uint32_t a[4], b[4];
        a[0] = pack_bf16(s[0][0], s[0][1]); a[1] = pack_bf16(s[0][2], s[0][3]);
        a[2] = pack_bf16(s[1][0], s[1][1]); a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int jj = 0; jj < NV / 2; ++jj) {
            o[2 * jj][0] *= corr0; o[2 * jj][1] *= corr0; o[2 * jj][2] *= corr1; o[2 * jj][3] *= corr1;
            o[2 * jj + 1][0] *= corr0; o[2 * jj + 1][1] *= corr0; o[2 * jj + 1][2] *= corr1; o[2 * jj + 1][3] *= corr1;
            ldsm_x4_trans(b, vb + 16 * jj * 2);
            mma_bf16(o[2 * jj], a, b[0], b[1]);
            mma_bf16(o[2 * jj + 1], a, b[2], b[3]);
        }
        __syncthreads();
    }
    // the four warps' shares of the keys are put together through shared memory: [warp][row][max, sum, dv lanes]
    l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
    l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
    l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
    l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
    float* sh = reinterpret_cast<float*>(Kb);          // the page buffers are done with (the loop ended on a barrier)
    const int rstride = 8 * NV + 2;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = quad + 8 * half;
        float* dst = sh + ((size_t)warp * 16 + r) * rstride;
        if (pair == 0) {
            dst[0] = m[half];
            dst[1] = l[half];
        }
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            dst[2 + 8 * j + pair] = o[j][2 * half];
            dst[2 + 8 * j + pair + 1] = o[j][2 * half + 1];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < group * dv; idx += 128) {
        const int r = idx / dv, d = idx % dv;
        float big = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) big = fmaxf(big, sh[((size_t)w * 16 + r) * rstride]);
        float lsum = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float* src = sh + ((size_t)w * 16 + r) * rstride;
            if (src[0] > -INFINITY) {
                const float f = fast_exp2(src[0] - big);
                lsum += src[1] * f;
                acc += src[2 + d] * f;
            }
        }
        const int head = head0 + r;
        if (n_splits > 1) {
            float* part = partial + (((size_t)n * n_heads + head) * n_splits + split) * (dv + 2);
            if (d == 0) {
                part[0] = big * 0.6931471805599453f;       // the splits are put together in natural units
                part[1] = lsum;
            }
            part[2 + d] = acc;
        } else {
            const float g = gate ? 1.0f / (1.0f + expf(-gate[(size_t)n * gate_stride + head])) : 1.f;
            out[((size_t)n * n_heads + head) * dv + d] = __float2bfloat16_rn(lsum > 0.f ? acc * g / lsum : 0.f);
        }
    }
}

template <int NV, int kDecodeStages>
static int launch_decode(const void* q, const void* pool, long long page_elems, const int* block_table, int table_stride,
                         const int* token_seq, const int* token_pos, const int* slot_of_seq, const float* gate, long long gate_stride,
                         void* out, float* partial, int n_splits, int n_tokens, int n_heads, int n_kv, int dk, int dv, int window,
                         int keep_first, float scale, int sink, ScoreOpts so, cudaStream_t stream) {
    const int dkp = (dk + 15) & ~15;
    size_t smem = ((size_t)16 * (dkp + 8) + (size_t)kDecodeStages * kTileK * ((dkp + 8) + (8 * NV + 8))) * sizeof(__nv_bfloat16);
    const size_t merge = (size_t)16 * (dkp + 8) * sizeof(__nv_bfloat16) + (size_t)4 * 16 * (8 * NV + 2) * sizeof(float);
    if (merge > smem) smem = merge;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attention_sink_decode_kernel<NV, kDecodeStages>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "attention_sink: %s", cudaGetErrorString(e));
    }
    cudaFuncSetAttribute(attention_sink_decode_kernel<NV, kDecodeStages>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    attention_sink_decode_kernel<NV, kDecodeStages><<<dim3(n_tokens, n_kv, n_splits), 128, smem, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)pool, page_elems, block_table, table_stride, token_seq, token_pos, slot_of_seq, gate,
        gate_stride, (__nv_bfloat16*)out, partial, n_heads, n_kv, dk, dv, window, keep_first, scale, sink, so);
    if (n_splits > 1) {
        const int items = n_tokens * n_heads;
        attention_sink_combine_kernel<__nv_bfloat16><<<(items + 3) / 4, 128, 0, stream>>>(partial, gate, gate_stride, (__nv_bfloat16*)out,
                                                                                         n_tokens, n_heads, dv, n_splits);
    }
    return blm_check_launch("attention_sink (decode)");
}

// How many query heads of a group share a block of the prompt kernel (and with it every page of keys and values that
// the block brings in; the block's warps are four to a head), and how many pages it holds in shared memory (one worked
// on, the others on their way).  Measured on one 2,048-token prompt, 32 heads on 8 kv heads, window 1,024, heads of 64
// and of 128 lanes: one head and two pages 105 and 183 us; two heads 109 and 206; four heads 119 and 193; three
// pages 109 and 275; four pages 133 and 270.  So one head and two pages it is; the others build with
// -DBLM_PROMPT_HEADS=2|4 and -DBLM_PROMPT_STAGES=3|4.
#ifndef BLM_PROMPT_HEADS
#define BLM_PROMPT_HEADS 1
#endif
template <int NV, typename... Args>
static int launch_prompt_heads(int hb, Args... args) {
#if BLM_PROMPT_HEADS >= 4
    if (hb == 4) return launch_prompt<NV, 4>(args...);
#endif
#if BLM_PROMPT_HEADS >= 2
    if (hb >= 2) return launch_prompt<NV, 2>(args...);
#endif
    (void)hb;
    return launch_prompt<NV, 1>(args...);
}

// Whether a step of this shape runs the prompt kernel (else the row kernel): bfloat16, pages of 64, sizes it takes,
// and portions long enough to fill some of a tile's rows.
BLM_API int blm_attention_sink_prompt_takes(int dtype, int dk, int dv, int page_size, int max_q_len, int n_heads) {
    return dtype == BLM_BF16 && page_size == kTileK && dk % 8 == 0 && dv % 8 == 0 && dk >= 8 && dk <= 256 && dv >= 8 && dv <= 128 &&
           max_q_len >= 8 && n_heads <= 65535;
}

// Whether single tokens and short portions of this shape run the tensor-core decode kernel (else the row kernel): the
// same sizes, and a group of query heads that fits the 16 rows of a tile.  The keys are then cut by pages: a split
// should have a page at least.
BLM_API int blm_attention_sink_decode_takes(int dtype, int dk, int dv, int page_size, int n_heads, int n_kv) {
    return dtype == BLM_BF16 && page_size == kTileK && dk % 8 == 0 && dv % 8 == 0 && dk >= 8 && dk <= 256 && dv >= 8 && dv <= 128 &&
           n_kv > 0 && n_heads % n_kv == 0 && n_heads / n_kv <= 16;
}

BLM_API int blm_attention_sink(const void* q, const void* pool, int dtype, long long page_elems, const int* block_table,
                               int table_stride, const int* token_seq, const int* token_pos, const int* slot_of_seq,
                               const int* cu_seqlens, const int* start_pos, int n_seqs, int max_q_len, const float* gate,
                               long long gate_stride, void* out, float* partial, int n_splits, int n_tokens, int n_heads, int n_kv,
                               int dk, int dv, int page_size, int window, int keep_first, float scale, int sink,
                               const float* head_scale, const float* sink_logit, float softcap, cudaStream_t stream) {
    // head_scale, sink_logit: float32 [n_heads] or null; softcap: 0 for none (see ScoreOpts)
    if (n_tokens == 0) return BLM_OK;
    const ScoreOpts so{head_scale, sink_logit, softcap};
    BLM_REQUIRE(softcap >= 0.f, "attention_sink: a cap of %g", (double)softcap);
    BLM_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv > 0 && n_heads % n_kv == 0 && dk > 0 && dv > 0 && page_size > 0,
                "attention_sink: bad sizes");
    BLM_REQUIRE(dv <= 32 * kMaxVRegs, "attention_sink: values of %d lanes; at most %d", dv, 32 * kMaxVRegs);
    BLM_REQUIRE(window >= 1 && keep_first >= 0, "attention_sink: window %d, kept first %d", window, keep_first);
    BLM_REQUIRE(page_elems == (long long)n_kv * page_size * (dk + dv), "attention_sink: a page holds n_kv * page * (dk + dv) elements");
    BLM_REQUIRE(n_kv <= 65535 && n_splits >= 1 && n_splits <= 65535, "attention_sink: %d kv heads, %d splits", n_kv, n_splits);
    BLM_REQUIRE(n_splits == 1 || partial != nullptr, "attention_sink: %d splits need scratch", n_splits);
    if (cu_seqlens != nullptr && start_pos != nullptr && n_seqs > 0 &&
        blm_attention_sink_prompt_takes(dtype, dk, dv, page_size, max_q_len, n_heads)) {
#define BLM_PROMPT(NV) launch_prompt_heads<NV>(hb, q, pool, page_elems, block_table, table_stride, cu_seqlens, start_pos, slot_of_seq, n_seqs, gate, \
                                         gate_stride, out, n_tokens, n_heads, n_kv, dk, dv, window, keep_first, scale, sink, so, stream)
        const int group = n_heads / n_kv;
        int hb = BLM_PROMPT_HEADS;
        while (hb > 1 && (group % hb != 0 || (hb == 4 && dv > 64))) hb /= 2;    // four heads of 128 lanes would not fit the registers
        if (dv <= 32) return BLM_PROMPT(4);
        if (dv <= 64) return BLM_PROMPT(8);
        return BLM_PROMPT(16);
#undef BLM_PROMPT
    }
    if (blm_attention_sink_decode_takes(dtype, dk, dv, page_size, n_heads, n_kv)) {
#define BLM_DECODE(NV, STAGES) launch_decode<NV, STAGES>(q, pool, page_elems, block_table, table_stride, token_seq, token_pos, slot_of_seq, gate, gate_stride, \
                                         out, partial, n_splits, n_tokens, n_heads, n_kv, dk, dv, window, keep_first, scale, sink, so, stream)
        if (dv <= 32) return BLM_DECODE(4, 2);
        if (dv <= 64) return BLM_DECODE(8, 2);
        return BLM_DECODE(16, 3);
#undef BLM_DECODE
    }
    if (dtype == BLM_F32)
        return launch_rows<float>(q, pool, page_elems, block_table, table_stride, token_seq, token_pos, slot_of_seq, gate, gate_stride,
                                  out, partial, n_splits, n_tokens, n_heads, n_kv, dk, dv, page_size, window, keep_first, scale, sink,
                                  so, stream);
    if (dtype == BLM_BF16)
        return launch_rows<__nv_bfloat16>(q, pool, page_elems, block_table, table_stride, token_seq, token_pos, slot_of_seq, gate,
                                          gate_stride, out, partial, n_splits, n_tokens, n_heads, n_kv, dk, dv, page_size, window,
                                          keep_first, scale, sink, so, stream);
    return blm_fail(BLM_BAD_ARGUMENT, "attention_sink: dtype %d", dtype);
}
