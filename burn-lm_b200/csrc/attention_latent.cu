// Attention over a cached latent: every position keeps one normed latent vector c [R] and one rotated key part k_rot [dr]
// shared by all heads, nothing per head.  A head's key is [W_uk,h c | k_rot] and its value W_uv,h c; because both are linear
// in c, the up-projections are moved off the keys: with q' = W_uk,h^T q_nope the score is (q' . c + q_rot . k_rot) * scale, and
// the output is W_uv,h (sum_j p_j c_j).  So the kernel below is attention of H query heads on ONE key of R + dr lanes per
// position whose first R lanes are also the value; the two small products per head (q' before, W_uv after) are batched
// matrix products outside it.
//
//   blm_latent_prepare    q projection -> q_nope [H][N][dk] (the batched product's operand) and rotated q_rot [N][H][dr];
//                         down projection -> RMS-normed c and rotated k_rot, appended to the token's place in the cache
//   blm_latent_attention  causal softmax attention of a step's rows over the cache, keys cut over `splits` blocks; options:
//                         a window (position i sees j with 0 <= i - j < window) and a sink per head (one more entry
//                         exp(sink_h) in the softmax's denominator, without a key or a value, not scaled)
//   blm_latent_gather     the pages of a step's sequences, copied side by side in the order of the sequences
//   blm_latent_expand     keys and values of every head, made from gathered latents, laid out as pages of the
//                         grouped-query attention kernels ([2][heads][page_size][hd]): long prompts run those
//   blm_sigmoid_gate      out = o * sigmoid(g)
//
// Cache page: [page_size][R + dr] in the cache's dtype.  Scores, softmax and sums are fp32 in both dtypes.
#include "common.cuh"

BLM_API const char* blm_attention_latent_last_error() { return g_blm_error; }

// lanes 2i and 2i + 1 of a rotated part (`halves`: lanes i and i + rot_dims / 2) turn by pos * freq[i]; lanes from rot_dims
// on pass unchanged.  The angle, its sine and cosine are taken in fp64 and applied in fp32.
// `turn`: (cosine, sine) of the token's angle for every pair, worked out once a token (the heads and the key part turn alike)
__device__ __forceinline__ float rotated_lane(const float* src, int j, int rot_dims, const float2* __restrict__ turn, int halves) {
    if (j >= rot_dims) return src[j];
    const int half = rot_dims >> 1;
    const int i = halves ? (j < half ? j : j - half) : (j >> 1);
    const int ia = halves ? i : 2 * i, ib = halves ? i + half : 2 * i + 1;
    const float a = src[ia], b = src[ib], cf = turn[i].x, sf = turn[i].y;
    return j == ib ? b * cf + a * sf : a * cf - b * sf;
}

template <typename T>
__global__ void latent_prepare_kernel(const float* __restrict__ qp, long long qp_stride, const float* __restrict__ dkv,
                                      long long dkv_stride, const float* __restrict__ c_weight, float eps,
                                      const double* __restrict__ freq, int rot_dims, T* __restrict__ q_nope,
                                      float* __restrict__ q_rot, T* __restrict__ q_full, int hd_full, T* __restrict__ pool,
                                      const int* __restrict__ token_seq,
                                      const int* __restrict__ token_pos, const int* __restrict__ slot_of_seq,
                                      const int* __restrict__ block_table, int table_stride, int n_tokens, int H, int dk, int dr,
                                      int R, int page_size, int halves) {
    __shared__ float red[33];
    extern __shared__ float2 turn[];            // [rot_dims / 2]
    const int n = blockIdx.x;
    const int seq = token_seq[n];
    const bool real = seq >= 0;                 // a row of no sequence leaves zeros and reaches no cache
    const int pos = real ? token_pos[n] : 0;
    for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
        double sn, cs;
        sincos((double)pos * freq[i], &sn, &cs);
        turn[i] = make_float2((float)cs, (float)sn);
    }
    __syncthreads();
    const float* qrow = qp + (size_t)n * qp_stride;
    if (q_full != nullptr) {                    // whole heads [unrotated | rotated | zeros up to hd_full], for the expanded keys
        for (int idx = threadIdx.x; idx < H * hd_full; idx += blockDim.x) {
            const int h = idx / hd_full, d = idx % hd_full;
            float v = 0.f;
            if (real && d < dk) v = qrow[(size_t)h * (dk + dr) + d];
            else if (real && d < dk + dr) v = rotated_lane(qrow + (size_t)h * (dk + dr) + dk, d - dk, rot_dims, turn, halves);
            q_full[((size_t)n * H + h) * hd_full + d] = from_f32<T>(v);
        }
    }
    for (int idx = threadIdx.x; q_full == nullptr && idx < H * dk; idx += blockDim.x) {
        const int h = idx / dk, d = idx % dk;
        q_nope[((size_t)h * n_tokens + n) * dk + d] = from_f32<T>(real ? qrow[(size_t)h * (dk + dr) + d] : 0.f);
    }
    for (int idx = threadIdx.x; q_full == nullptr && idx < H * dr; idx += blockDim.x) {
        const int h = idx / dr, j = idx % dr;
        q_rot[((size_t)n * H + h) * dr + j] = real ? rotated_lane(qrow + (size_t)h * (dk + dr) + dk, j, rot_dims, turn, halves) : 0.f;
    }
    if (!real) return;
    const float* row = dkv + (size_t)n * dkv_stride;
    float ss = 0.f;
    for (int r = threadIdx.x; r < R; r += blockDim.x) ss += row[r] * row[r];
    const float total = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(total / (float)R + eps);
    const int page = block_table[(size_t)slot_of_seq[seq] * table_stride + pos / page_size];
    T* dst = pool + ((size_t)page * page_size + pos % page_size) * (R + dr);
    for (int r = threadIdx.x; r < R; r += blockDim.x) dst[r] = from_f32<T>(row[r] * inv * c_weight[r]);
    for (int j = threadIdx.x; j < dr; j += blockDim.x) dst[R + j] = from_f32<T>(rotated_lane(row + R, j, rot_dims, turn, halves));
}

BLM_API int blm_latent_prepare(const float* qp, long long qp_stride, const float* dkv, long long dkv_stride, const float* c_weight,
                               float eps, const double* freq, int rot_dims, void* q_nope, float* q_rot, void* q_full, int hd_full,
                               void* pool, int dtype,
                               const int* token_seq, const int* token_pos, const int* slot_of_seq, const int* block_table,
                               int table_stride, int n_tokens, int H, int dk, int dr, int R, int page_size, int halves,
                               cudaStream_t stream) {
    // halves 0: the turning lanes are paired (2i, 2i + 1); 1: (i, i + rot_dims / 2)
    if (n_tokens == 0) return BLM_OK;
    BLM_REQUIRE(H > 0 && dk > 0 && dr >= 0 && R > 0 && page_size > 0, "latent_prepare: bad sizes");
    BLM_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dr, "latent_prepare: %d rotated lanes of %d", rot_dims, dr);
    BLM_REQUIRE(q_full != nullptr ? hd_full >= dk + dr : (q_nope != nullptr && q_rot != nullptr),
                "latent_prepare: whole heads of at least %d lanes, or the two parts", dk + dr);
    if (dtype == BLM_F32)
        latent_prepare_kernel<float><<<n_tokens, 256, (size_t)(rot_dims / 2 + 1) * sizeof(float2), stream>>>(qp, qp_stride, dkv, dkv_stride, c_weight, eps, freq, rot_dims,
                                                                   (float*)q_nope, q_rot, (float*)q_full, hd_full, (float*)pool, token_seq, token_pos,
                                                                   slot_of_seq, block_table, table_stride, n_tokens, H, dk, dr, R,
                                                                   page_size, halves);
    else if (dtype == BLM_BF16)
        latent_prepare_kernel<__nv_bfloat16><<<n_tokens, 256, (size_t)(rot_dims / 2 + 1) * sizeof(float2), stream>>>(qp, qp_stride, dkv, dkv_stride, c_weight, eps, freq, rot_dims,
                                                                           (__nv_bfloat16*)q_nope, q_rot, (__nv_bfloat16*)q_full, hd_full, (__nv_bfloat16*)pool,
                                                                           token_seq, token_pos, slot_of_seq, block_table,
                                                                           table_stride, n_tokens, H, dk, dr, R, page_size, halves);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "latent_prepare: dtype %d", dtype);
    return blm_check_launch("latent_prepare");
}

// ---------------------------------------------------------------------------------------------
// attention.  A block owns kTM rows of one sequence (row = new token x head, the heads of a token side by side: they
// all read the same keys) and one share of the keys; keys pass through shared memory kKC at a time, in fp32.  Thread t
// holds the output columns t, t + 256, ... of all kTM rows.
// ---------------------------------------------------------------------------------------------
constexpr int kTM = 16, kKC = 32, kLatThreads = 256;

template <typename T, typename TO, int CPT>
__global__ void __launch_bounds__(kLatThreads)
    latent_attention_kernel(const float* __restrict__ q_lat, const float* __restrict__ q_rot, const T* __restrict__ pool,
                            const int* __restrict__ block_table, int table_stride, const int* __restrict__ cu_seqlens,
                            const int* __restrict__ slot_of_seq, const int* __restrict__ start_pos, TO* __restrict__ out,
                            float* __restrict__ partial, int n_tokens, int H, int R, int dr, int page_size, float scale,
                            int n_splits, int window, const float* __restrict__ sink) {
    const int seq = blockIdx.y, split = blockIdx.z;
    const int first = cu_seqlens[seq];
    const int n_new = cu_seqlens[seq + 1] - first;
    if (n_new <= 0) return;
    const int rows_total = n_new * H, r0 = blockIdx.x * kTM;
    if (r0 >= rows_total) return;
    const int n_rows = min(kTM, rows_total - r0);
    const int start = start_pos[seq];
    const int kv_end = start + (r0 + n_rows - 1) / H + 1;          // keys the tile's last row sees
    // the tile's first row sees no key before its window: the walk starts at that key's page (window 0: at the first page)
    const int page_lo = window > 0 ? max(0, start + r0 / H - window + 1) / page_size : 0;
    const int pages_total = (kv_end + page_size - 1) / page_size - page_lo;
    const int pages_per = (pages_total + n_splits - 1) / n_splits;
    const int key_lo = min(kv_end, (page_lo + split * pages_per) * page_size);
    const int key_hi = min(kv_end, (page_lo + (split + 1) * pages_per) * page_size);
    const int D = R + dr, KS = D + 1;
    extern __shared__ __align__(16) float lat_smem[];
    float* Pt = lat_smem;                    // [kKC][kTM]: a chunk's weights, key by key
    float* Qs = Pt + kKC * kTM;              // [kTM][D]
    float* Ks = Qs + kTM * D;                // [kKC][D + 1]
    float* Ss = Ks + kKC * KS;               // [kTM][kKC]
    __shared__ float m_s[kTM], l_s[kTM], alpha_s[kTM];
    __shared__ int page_of[kKC];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int* table = block_table + (size_t)slot_of_seq[seq] * table_stride;
    for (int idx = tid; idx < kTM * D; idx += kLatThreads) {
        const int row = idx / D, d = idx % D;
        float v = 0.f;
        if (row < n_rows) {
            const int r = r0 + row, n = first + r / H, h = r % H;
            v = d < R ? q_lat[((size_t)h * n_tokens + n) * R + d] : q_rot[((size_t)n * H + h) * dr + (d - R)];
        }
        Qs[idx] = v;
    }
    if (tid < kTM) {                         // the sink is one more entry of the first share: a score without a value
        const bool with_sink = sink != nullptr && split == 0;
        m_s[tid] = with_sink ? sink[(r0 + tid) % H] : -INFINITY;
        l_s[tid] = with_sink ? 1.f : 0.f;
    }
    float acc[kTM][CPT];
#pragma unroll
    for (int r = 0; r < kTM; ++r)
#pragma unroll
        for (int c = 0; c < CPT; ++c) acc[r][c] = 0.f;
    for (int k0 = key_lo; k0 < key_hi; k0 += kKC) {
        const int nk = min(kKC, key_hi - k0);
        __syncthreads();                     // the chunk before is used up (and Qs, m_s, l_s are written)
        if (tid < kKC) page_of[tid] = tid < nk ? table[(k0 + tid) / page_size] : 0;
        __syncthreads();
        for (int idx = tid; idx < kKC * D; idx += kLatThreads) {
            const int j = idx / D, d = idx % D;
            float v = 0.f;
            if (j < nk) v = to_f32(pool[((size_t)page_of[j] * page_size + (k0 + j) % page_size) * D + d]);
            Ks[j * KS + d] = v;
        }
        __syncthreads();
        {                                    // scores: thread (row, key pair)
            const int row = tid >> 4, jp = tid & 15;
            const float* qr = Qs + row * D;
            const float* ka = Ks + jp * KS;
            const float* kb = Ks + (jp + 16) * KS;
            float sa = 0.f, sb = 0.f;
            for (int d = 0; d < D; ++d) {
                const float qv = qr[d];
                sa = fmaf(qv, ka[d], sa);
                sb = fmaf(qv, kb[d], sb);
            }
            const int limit = start + (r0 + row) / H;            // the row's own position
            const int from = window > 0 ? limit - window + 1 : 0; // the first key it sees
            const bool live = row < n_rows;
            Ss[row * kKC + jp] = (live && jp < nk && k0 + jp <= limit && k0 + jp >= from) ? sa * scale : -INFINITY;
            Ss[row * kKC + jp + 16] = (live && jp + 16 < nk && k0 + jp + 16 <= limit && k0 + jp + 16 >= from) ? sb * scale : -INFINITY;
        }
        __syncthreads();
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {     // running softmax: a warp takes two rows, a lane a key
            const int row = 2 * warp + rr;
            const float s = Ss[row * kKC + lane];
            const float m_old = m_s[row];
            const float m_new = fmaxf(m_old, warp_max(s));
            float p = 0.f, alpha = 1.f;
            if (m_new > -INFINITY) {
                p = s > -INFINITY ? expf(s - m_new) : 0.f;
                alpha = m_old > -INFINITY ? expf(m_old - m_new) : 0.f;
            }
            const float sum = warp_sum(p);
            Pt[lane * kTM + row] = p;
            if (lane == 0) {
                m_s[row] = m_new;
                l_s[row] = l_s[row] * alpha + sum;
                alpha_s[row] = alpha;
            }
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < kTM; ++r) {
            const float a = alpha_s[r];
#pragma unroll
            for (int c = 0; c < CPT; ++c) acc[r][c] *= a;
        }
        for (int j = 0; j < nk; ++j) {
            float p[kTM];
#pragma unroll
            for (int r4 = 0; r4 < kTM / 4; ++r4) {
                const float4 v = *reinterpret_cast<const float4*>(Pt + j * kTM + 4 * r4);
                p[4 * r4] = v.x; p[4 * r4 + 1] = v.y; p[4 * r4 + 2] = v.z; p[4 * r4 + 3] = v.w;
            }
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const int col = tid + c * kLatThreads;
                const float v = col < R ? Ks[j * KS + col] : 0.f;
#pragma unroll
                for (int r = 0; r < kTM; ++r) acc[r][c] = fmaf(p[r], v, acc[r][c]);
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kTM; ++r) {
        if (r >= n_rows) break;
        const int rr = r0 + r, n = first + rr / H, h = rr % H;
        if (n_splits == 1) {
            const float inv = 1.0f / l_s[r];
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const int col = tid + c * kLatThreads;
                if (col < R) out[((size_t)h * n_tokens + n) * R + col] = from_f32<TO>(acc[r][c] * inv);
            }
        } else {
            float* dst = partial + ((size_t)split * n_tokens * H + (size_t)n * H + h) * (R + 2);
            if (tid == 0) {
                dst[0] = m_s[r];
                dst[1] = l_s[r];
            }
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const int col = tid + c * kLatThreads;
                if (col < R) dst[2 + col] = acc[r][c];
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The same attention with both products on the tensor cores (mma.sync m16n8k16, bfloat16 operands, fp32 sums), for a
// bfloat16 cache whose latent and rotated part are multiples of 16 lanes.  A block owns 16 MT rows and a share of the
// keys; a chunk of 32 keys lies in shared memory once, as it is cached, and serves as B operand of both products:
// as it lies for the scores (lanes are the contraction), read transposed for the sums (keys are).  Eight warps:
//   scores  warp = (8 keys of the chunk, one half of the lanes), all row tiles; the halves meet in the softmax
//   softmax a warp takes 2 MT rows, a lane a key; weights go to shared memory as bfloat16, sums stay fp32
//   sums    a warp owns 8 NT output columns of all rows, in registers
// ---------------------------------------------------------------------------------------------
namespace lat {
constexpr int KC = 32, THREADS = 256, SS = KC + 8, PS = KC + 8;
__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x2(unsigned& r0, unsigned& r1, const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async_16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }
__host__ __device__ inline size_t smem_bytes(int rows, int D) {
    return ((size_t)rows * (D + 8) + (size_t)KC * (D + 8) + (size_t)rows * PS) * sizeof(__nv_bfloat16) + (size_t)2 * rows * SS * sizeof(float);
}
}  // namespace lat

template <typename TO, int MT, int NT>
__global__ void __launch_bounds__(lat::THREADS, 2)
    latent_attention_mma_kernel(const float* __restrict__ q_lat, const float* __restrict__ q_rot, const __nv_bfloat16* __restrict__ pool,
                                const int* __restrict__ block_table, int table_stride, const int* __restrict__ cu_seqlens,
                                const int* __restrict__ slot_of_seq, const int* __restrict__ start_pos, TO* __restrict__ out,
                                float* __restrict__ partial, int n_tokens, int H, int R, int dr, int page_size, float scale,
                                int n_splits, int window, const float* __restrict__ sink) {
    using namespace lat;
    constexpr int ROWS = 16 * MT;
    const int seq = blockIdx.y, split = blockIdx.z;
    const int first = cu_seqlens[seq];
    const int n_new = cu_seqlens[seq + 1] - first;
    if (n_new <= 0) return;
    const int rows_total = n_new * H, r0 = blockIdx.x * ROWS;
    if (r0 >= rows_total) return;
    const int n_rows = min(ROWS, rows_total - r0);
    const int start = start_pos[seq];
    const int kv_end = start + (r0 + n_rows - 1) / H + 1;          // keys the tile's last row sees
    const int page_lo = window > 0 ? max(0, start + r0 / H - window + 1) / page_size : 0;   // as in the kernel above
    const int pages_total = (kv_end + page_size - 1) / page_size - page_lo;
    const int pages_per = (pages_total + n_splits - 1) / n_splits;
    const int key_lo = min(kv_end, (page_lo + split * pages_per) * page_size);
    const int key_hi = min(kv_end, (page_lo + (split + 1) * pages_per) * page_size);
    const int D = R + dr, LD = D + 8;
    extern __shared__ __align__(16) unsigned char lat_mma_smem[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(lat_mma_smem);      // [ROWS][LD]
    __nv_bfloat16* Ks = Qs + ROWS * LD;                                      // [KC][LD]
    __nv_bfloat16* Ps = Ks + KC * LD;                                        // [ROWS][PS]
    float* Ss = reinterpret_cast<float*>(Ps + ROWS * PS);                    // [2][ROWS][SS]: the two halves of the lanes
    __shared__ float m_s[ROWS], l_s[ROWS], alpha_s[ROWS];
    __shared__ int page_of[KC];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int* table = block_table + (size_t)slot_of_seq[seq] * table_stride;
    for (int row = warp; row < ROWS; row += THREADS / 32) {      // a warp a row: no division an element, loads side by side
        const int r = r0 + row, n = first + r / H, h = r % H;
        const float* lat_row = q_lat + ((size_t)h * n_tokens + n) * R;
        const float* rot_row = q_rot + ((size_t)n * H + h) * dr;
#pragma unroll 4
        for (int d = lane; d < D; d += 32) {
            float v = 0.f;
            if (row < n_rows) v = d < R ? lat_row[d] : rot_row[d - R];
            Qs[row * LD + d] = __float2bfloat16(v);
        }
    }
    if (tid < ROWS) {
        const bool with_sink = sink != nullptr && split == 0;
        m_s[tid] = with_sink ? sink[(r0 + tid) % H] : -INFINITY;
        l_s[tid] = with_sink ? 1.f : 0.f;
    }
    float acc[MT][NT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[m][n][i] = 0.f;
    const int vecs = D / 8, ksteps = D / 16;
    for (int k0 = key_lo; k0 < key_hi; k0 += KC) {
        const int nk = min(KC, key_hi - k0);
        __syncthreads();                     // the chunk before is used up (and Qs, m_s, l_s are written)
        if (tid < KC) page_of[tid] = tid < nk ? table[(k0 + tid) / page_size] : 0;
        __syncthreads();
        for (int idx = tid; idx < KC * vecs; idx += THREADS) {   // asynchronous copies: all of a thread's pieces are on their way at once
            const int j = idx / vecs, c = idx - j * vecs;
            __nv_bfloat16* dst = Ks + j * LD + c * 8;
            if (j < nk)
                cp_async_16(dst, pool + ((size_t)page_of[j] * page_size + (k0 + j) % page_size) * D + c * 8);
            else
                *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);   // keys beyond the share are zeros: a weight of 0 silences no NaN
        }
        cp_async_wait_all();
        __syncthreads();
        {                                    // scores
            const int nt = warp & 3, half = warp >> 2;
            const int ks_lo = half ? (ksteps + 1) / 2 : 0, ks_hi = half ? ksteps : (ksteps + 1) / 2;
            float c[MT][4];
#pragma unroll
            for (int m = 0; m < MT; ++m) c[m][0] = c[m][1] = c[m][2] = c[m][3] = 0.f;
            for (int ks = ks_lo; ks < ks_hi; ++ks) {
                unsigned b0, b1;
                ldsm_x2(b0, b1, Ks + (nt * 8 + (lane & 7)) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    unsigned a[4];
                    ldsm_x4(a, Qs + (m * 16 + (lane & 15)) * LD + ks * 16 + (lane >> 4) * 8);
                    mma_bf16(c[m], a, b0, b1);
                }
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                float* dst = Ss + ((size_t)half * ROWS + m * 16 + g) * SS + nt * 8 + 2 * t;
                *reinterpret_cast<float2*>(dst) = make_float2(c[m][0], c[m][1]);
                *reinterpret_cast<float2*>(dst + 8 * SS) = make_float2(c[m][2], c[m][3]);
            }
        }
        __syncthreads();
#pragma unroll
        for (int rr = 0; rr < 2 * MT; ++rr) {     // running softmax: a warp takes 2 MT rows, a lane a key
            const int row = 2 * MT * warp + rr;
            const int limit = start + (r0 + row) / H;
            const bool seen = row < n_rows && lane < nk && k0 + lane <= limit && (window <= 0 || k0 + lane > limit - window);
            const float s = seen ? (Ss[row * SS + lane] + Ss[(ROWS + row) * SS + lane]) * scale : -INFINITY;
            const float m_old = m_s[row];
            const float m_new = fmaxf(m_old, warp_max(s));
            float p = 0.f, alpha = 1.f;
            if (m_new > -INFINITY) {
                p = s > -INFINITY ? expf(s - m_new) : 0.f;
                alpha = m_old > -INFINITY ? expf(m_old - m_new) : 0.f;
            }
            const float sum = warp_sum(p);
            Ps[row * PS + lane] = __float2bfloat16(p);
            if (lane == 0) {
                m_s[row] = m_new;
                l_s[row] = l_s[row] * alpha + sum;
                alpha_s[row] = alpha;
            }
        }
        __syncthreads();
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const float lo = alpha_s[m * 16 + g], hi = alpha_s[m * 16 + g + 8];
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                acc[m][n][0] *= lo; acc[m][n][1] *= lo; acc[m][n][2] *= hi; acc[m][n][3] *= hi;
            }
        }
#pragma unroll
        for (int kk = 0; kk < KC / 16; ++kk) {
            unsigned a[MT][4];
#pragma unroll
            for (int m = 0; m < MT; ++m) ldsm_x4(a[m], Ps + (m * 16 + (lane & 15)) * PS + kk * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                const int n0 = (warp * NT + 2 * np) * 8;
                if (n0 < R) {                // R is a multiple of 16: a pair of column tiles is inside or outside
                    unsigned b[4];
                    ldsm_x4_trans(b, Ks + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + n0 + (lane >> 4) * 8);
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        mma_bf16(acc[m][2 * np], a[m], b[0], b[1]);
                        mma_bf16(acc[m][2 * np + 1], a[m], b[2], b[3]);
                    }
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int row = m * 16 + g + 8 * hh;
            if (row >= n_rows) continue;
            const int rr = r0 + row, n = first + rr / H, h = rr % H;
            if (n_splits == 1) {
                const float inv = 1.0f / l_s[row];
#pragma unroll
                for (int nn = 0; nn < NT; ++nn) {
                    const int col = (warp * NT + nn) * 8 + 2 * t;
                    if (col < R) {
                        TO* dst = out + ((size_t)h * n_tokens + n) * R + col;
                        dst[0] = from_f32<TO>(acc[m][nn][2 * hh] * inv);
                        dst[1] = from_f32<TO>(acc[m][nn][2 * hh + 1] * inv);
                    }
                }
            } else {
                float* dst = partial + ((size_t)split * n_tokens * H + (size_t)n * H + h) * (R + 2);
                if (warp == 0 && t == 0) {
                    dst[0] = m_s[row];
                    dst[1] = l_s[row];
                }
#pragma unroll
                for (int nn = 0; nn < NT; ++nn) {
                    const int col = (warp * NT + nn) * 8 + 2 * t;
                    if (col < R) {
                        dst[2 + col] = acc[m][nn][2 * hh];
                        dst[2 + col + 1] = acc[m][nn][2 * hh + 1];
                    }
                }
            }
        }
}

// rows (token x head) of a block: 16 on the CUDA cores; 16 or 32 on the tensor cores
static bool latent_takes_mma(int dtype, int R, int dr) { return dtype == BLM_BF16 && R % 16 == 0 && dr % 16 == 0 && R <= 512; }
BLM_API int blm_latent_attention_tile_rows(int dtype, int H, int R, int dr, int max_q_len) {
    if (!latent_takes_mma(dtype, R, dr)) return kTM;
    return (long long)max_q_len * H > 16 ? 32 : 16;
}

// the shares of a row's keys, merged in the order of the shares
template <typename TO>
__global__ void latent_combine_kernel(const float* __restrict__ partial, const int* __restrict__ token_seq, TO* __restrict__ out,
                                      int n_tokens, int H, int R, int n_splits) {
    const int n = blockIdx.x / H, h = blockIdx.x % H;
    if (token_seq[n] < 0) return;            // a row of no sequence: nothing was written for it, the caller's zeros stay
    const size_t stride = (size_t)n_tokens * H * (R + 2);
    const float* src = partial + ((size_t)n * H + h) * (R + 2);
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, src[s * stride]);
    float l = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = src[s * stride];
        if (ms > -INFINITY) l += src[s * stride + 1] * expf(ms - m);
    }
    const float inv = 1.0f / l;
    for (int c = threadIdx.x; c < R; c += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = src[s * stride];
            if (ms > -INFINITY) o += src[s * stride + 2 + c] * expf(ms - m);
        }
        out[((size_t)h * n_tokens + n) * R + c] = from_f32<TO>(o * inv);
    }
}

BLM_API long long blm_latent_attention_scratch_floats(int n_tokens, int H, int R, int n_splits) {
    return n_splits > 1 ? (long long)n_splits * n_tokens * H * (R + 2) : 0;
}

// q_lat float32 [H][N][R], q_rot float32 [N][H][dr]; out [H][N][R] in `out_dtype` (rows of no sequence are left alone);
// partial: float32 scratch of blm_latent_attention_scratch_floats when n_splits > 1.
BLM_API int blm_latent_attention(const float* q_lat, const float* q_rot, const void* pool, int dtype, const int* block_table,
                                 int table_stride, const int* cu_seqlens, const int* slot_of_seq, const int* start_pos,
                                 const int* token_seq, void* out, int out_dtype, float* partial, int n_tokens, int n_seqs,
                                 int max_q_len, int H, int R, int dr, int page_size, float scale, int n_splits, int window,
                                 const float* sink, cudaStream_t stream) {
    // window: 0 for every earlier key; sink: float32 [H] or null
    if (n_tokens == 0 || n_seqs == 0) return BLM_OK;
    BLM_REQUIRE(H > 0 && R > 0 && dr >= 0 && page_size > 0 && max_q_len > 0 && n_splits >= 1, "latent_attention: bad sizes");
    BLM_REQUIRE(R <= 4 * kLatThreads, "latent_attention: a latent of %d lanes; this kernel takes up to %d", R, 4 * kLatThreads);
    BLM_REQUIRE(n_splits == 1 || partial != nullptr, "latent_attention: key shares need their scratch");
    BLM_REQUIRE(window >= 0, "latent_attention: a window of %d", window);
    const int D = R + dr;
    if (latent_takes_mma(dtype, R, dr) && (out_dtype == BLM_BF16 || out_dtype == BLM_F32) && ((size_t)pool & 15) == 0) {
        const int rows = blm_latent_attention_tile_rows(dtype, H, R, dr, max_q_len);
        const size_t smem = lat::smem_bytes(rows, D);
        const long long tiles = ((long long)max_q_len * H + rows - 1) / rows;
        BLM_REQUIRE(tiles < (1ll << 31) && n_seqs <= 65535 && n_splits <= 65535, "latent_attention: too many blocks");
        const dim3 grid((unsigned)tiles, (unsigned)n_seqs, (unsigned)n_splits);
        const int nt = R <= 128 ? 2 : R <= 256 ? 4 : 8;
#define BLM_LAT_MMA(TO, MT, NT)                                                                                          \
    {                                                                                                                    \
        auto kern = latent_attention_mma_kernel<TO, MT, NT>;                                                             \
        if (smem > 48 * 1024) {                                                                                          \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
            if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "latent_attention: %s", cudaGetErrorString(e));        \
        }                                                                                                                \
        kern<<<grid, lat::THREADS, smem, stream>>>(q_lat, q_rot, (const __nv_bfloat16*)pool, block_table, table_stride,  \
                                                   cu_seqlens, slot_of_seq, start_pos, (TO*)out, partial, n_tokens, H,   \
                                                   R, dr, page_size, scale, n_splits, window, sink);                     \
    }
#define BLM_LAT_MMA_N(TO, MT)                                            \
    if (nt == 2) BLM_LAT_MMA(TO, MT, 2)                                  \
    else if (nt == 4) BLM_LAT_MMA(TO, MT, 4)                             \
    else BLM_LAT_MMA(TO, MT, 8)
        if (out_dtype == BLM_BF16) {
            if (rows == 32) { BLM_LAT_MMA_N(__nv_bfloat16, 2) } else { BLM_LAT_MMA_N(__nv_bfloat16, 1) }
        } else {
            if (rows == 32) { BLM_LAT_MMA_N(float, 2) } else { BLM_LAT_MMA_N(float, 1) }
        }
#undef BLM_LAT_MMA_N
#undef BLM_LAT_MMA
        int rc = blm_check_launch("latent_attention (tensor cores)");
        if (rc != BLM_OK || n_splits == 1) return rc;
        if (out_dtype == BLM_F32)
            latent_combine_kernel<float><<<n_tokens * H, 128, 0, stream>>>(partial, token_seq, (float*)out, n_tokens, H, R, n_splits);
        else
            latent_combine_kernel<__nv_bfloat16><<<n_tokens * H, 128, 0, stream>>>(partial, token_seq, (__nv_bfloat16*)out, n_tokens, H, R,
                                                                                  n_splits);
        return blm_check_launch("latent_attention (combine)");
    }
    const size_t smem = ((size_t)kKC * kTM + (size_t)kTM * D + (size_t)kKC * (D + 1) + (size_t)kTM * kKC) * sizeof(float);
    BLM_REQUIRE(smem <= 200 * 1024, "latent_attention: keys of %d lanes need %zu bytes of shared memory", D, smem);
    const long long tiles = ((long long)max_q_len * H + kTM - 1) / kTM;
    BLM_REQUIRE(tiles < (1ll << 31) && n_seqs <= 65535 && n_splits <= 65535, "latent_attention: too many blocks");
    const dim3 grid((unsigned)tiles, (unsigned)n_seqs, (unsigned)n_splits);
    const int cpt = (R + kLatThreads - 1) / kLatThreads;
#define BLM_LAT(T, TO, CPT)                                                                                              \
    {                                                                                                                    \
        auto kern = latent_attention_kernel<T, TO, CPT>;                                                                 \
        if (smem > 48 * 1024) {                                                                                          \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
            if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "latent_attention: %s", cudaGetErrorString(e));        \
        }                                                                                                                \
        kern<<<grid, kLatThreads, smem, stream>>>(q_lat, q_rot, (const T*)pool, block_table, table_stride, cu_seqlens,   \
                                                  slot_of_seq, start_pos, (TO*)out, partial, n_tokens, H, R, dr,         \
                                                  page_size, scale, n_splits, window, sink);                             \
    }
#define BLM_LAT_C(T, TO)                                                 \
    if (cpt == 1) BLM_LAT(T, TO, 1)                                      \
    else if (cpt == 2) BLM_LAT(T, TO, 2)                                 \
    else if (cpt == 3) BLM_LAT(T, TO, 3)                                 \
    else BLM_LAT(T, TO, 4)
    if (dtype == BLM_F32 && out_dtype == BLM_F32) { BLM_LAT_C(float, float) }
    else if (dtype == BLM_BF16 && out_dtype == BLM_BF16) { BLM_LAT_C(__nv_bfloat16, __nv_bfloat16) }
    else if (dtype == BLM_BF16 && out_dtype == BLM_F32) { BLM_LAT_C(__nv_bfloat16, float) }
    else return blm_fail(BLM_BAD_ARGUMENT, "latent_attention: dtypes %d/%d", dtype, out_dtype);
#undef BLM_LAT_C
#undef BLM_LAT
    int rc = blm_check_launch("latent_attention");
    if (rc != BLM_OK || n_splits == 1) return rc;
    if (out_dtype == BLM_F32)
        latent_combine_kernel<float><<<n_tokens * H, 128, 0, stream>>>(partial, token_seq, (float*)out, n_tokens, H, R, n_splits);
    else
        latent_combine_kernel<__nv_bfloat16><<<n_tokens * H, 128, 0, stream>>>(partial, token_seq, (__nv_bfloat16*)out, n_tokens, H, R,
                                                                              n_splits);
    return blm_check_launch("latent_attention (combine)");
}

// ---------------------------------------------------------------------------------------------
// Long prompts: the heads' keys and values are written out for the step (k_h = [W_uk,h c | k_rot], v_h = W_uv,h c, one
// product over the gathered latents) in the page layout of the grouped-query attention kernels, which then run with as
// many key/value heads as query heads.  The expanded pages live for the step only; the cache keeps the latent.
// ---------------------------------------------------------------------------------------------
// out [n_seqs * pages_each][page_size][D]: page p of sequence s is its p-th cached page; positions the sequence has not
// reached (the cache is never cleared) and pages beyond its end are zeros.
template <typename T>
__global__ void latent_gather_kernel(const T* __restrict__ pool, const int* __restrict__ block_table, int table_stride,
                                     const int* __restrict__ cu_seqlens, const int* __restrict__ slot_of_seq,
                                     const int* __restrict__ start_pos, T* __restrict__ out, int pages_each, int D, int page_size,
                                     int window) {
    const int p = blockIdx.x, seq = blockIdx.y;
    const int kv_len = start_pos[seq] + cu_seqlens[seq + 1] - cu_seqlens[seq];
    // pages that lie wholly before the window of the step's first token may have been given back: zeros for them
    const bool before = window > 0 && (p + 1) * page_size <= start_pos[seq] - window + 1;
    const int live = before ? 0 : min(page_size, kv_len - p * page_size);
    T* dst = out + ((size_t)seq * pages_each + p) * page_size * D;
    const T* src = live > 0 ? pool + (size_t)block_table[(size_t)slot_of_seq[seq] * table_stride + p] * page_size * D : nullptr;
    const int n_live = live > 0 ? live * D : 0, n_all = page_size * D;
    if ((D * sizeof(T)) % 16 == 0) {
        constexpr int V = 16 / sizeof(T);
        const uint4 zero = make_uint4(0, 0, 0, 0);
        for (int i = threadIdx.x * V; i < n_all; i += blockDim.x * V)
            *reinterpret_cast<uint4*>(dst + i) = i < n_live ? *reinterpret_cast<const uint4*>(src + i) : zero;
    } else {
        for (int i = threadIdx.x; i < n_all; i += blockDim.x) dst[i] = i < n_live ? src[i] : from_f32<T>(0.f);
    }
}

BLM_API int blm_latent_gather(const void* pool, int dtype, const int* block_table, int table_stride, const int* cu_seqlens,
                              const int* slot_of_seq, const int* start_pos, void* out, int n_seqs, int pages_each, int D,
                              int page_size, int window, cudaStream_t stream) {
    // window: 0, or the mixer's window: pages wholly before it are not read
    if (n_seqs == 0 || pages_each == 0) return BLM_OK;
    BLM_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && pages_each > 0 && D > 0 && page_size > 0, "latent_gather: bad sizes");
    BLM_REQUIRE(pages_each <= table_stride, "latent_gather: %d pages a sequence, the table has %d", pages_each, table_stride);
    BLM_REQUIRE((((size_t)pool | (size_t)out) & 15) == 0, "latent_gather: buffers must be 16-byte aligned");
    const dim3 grid(pages_each, n_seqs);
    if (dtype == BLM_BF16)
        latent_gather_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)pool, block_table, table_stride, cu_seqlens,
                                                                     slot_of_seq, start_pos, (__nv_bfloat16*)out, pages_each, D, page_size, window);
    else if (dtype == BLM_F32)
        latent_gather_kernel<float><<<grid, 256, 0, stream>>>((const float*)pool, block_table, table_stride, cu_seqlens, slot_of_seq,
                                                             start_pos, (float*)out, pages_each, D, page_size, window);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "latent_gather: dtype %d", dtype);
    return blm_check_launch("latent_gather");
}

// kv [rows][ld]: a gathered position's unrotated keys of all heads ([H][dk]) and then its values ([H][dv]);
// gathered [rows][R + dr] gives the rotated key part.  out [pages][2][H][page_size][hd], lanes beyond a head's own are zeros.
template <typename T>
__global__ void latent_expand_kernel(const T* __restrict__ kv, long long ld, const T* __restrict__ gathered, T* __restrict__ out, int H,
                                     int dk, int dr, int dv, int R, int hd, int page_size) {
    const int page = blockIdx.x, h = blockIdx.y;
    T* kd = out + (((size_t)page * 2 + 0) * H + h) * page_size * hd;
    T* vd = out + (((size_t)page * 2 + 1) * H + h) * page_size * hd;
    const T zero = from_f32<T>(0.f);
    for (int idx = threadIdx.x; idx < page_size * hd; idx += blockDim.x) {
        const int j = idx / hd, d = idx % hd;
        const size_t row = (size_t)page * page_size + j;
        T k = zero, v = zero;
        if (d < dk) k = kv[row * ld + (size_t)h * dk + d];
        else if (d < dk + dr) k = gathered[row * (R + dr) + R + (d - dk)];
        if (d < dv) v = kv[row * ld + (size_t)H * dk + (size_t)h * dv + d];
        kd[idx] = k;
        vd[idx] = v;
    }
}

BLM_API int blm_latent_expand(const void* kv, long long ld, const void* gathered, void* out, int dtype, int n_pages, int H, int dk,
                              int dr, int dv, int R, int hd, int page_size, cudaStream_t stream) {
    if (n_pages == 0) return BLM_OK;
    BLM_REQUIRE(n_pages > 0 && H > 0 && H <= 65535 && dk > 0 && dr >= 0 && dv > 0 && R > 0 && page_size > 0, "latent_expand: bad sizes");
    BLM_REQUIRE(hd >= dk + dr && hd >= dv, "latent_expand: heads of %d lanes for keys of %d and values of %d", hd, dk + dr, dv);
    const dim3 grid(n_pages, H);
    if (dtype == BLM_BF16)
        latent_expand_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)kv, ld, (const __nv_bfloat16*)gathered,
                                                                     (__nv_bfloat16*)out, H, dk, dr, dv, R, hd, page_size);
    else if (dtype == BLM_F32)
        latent_expand_kernel<float><<<grid, 256, 0, stream>>>((const float*)kv, ld, (const float*)gathered, (float*)out, H, dk, dr, dv, R,
                                                             hd, page_size);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "latent_expand: dtype %d", dtype);
    return blm_check_launch("latent_expand");
}

// ---------------------------------------------------------------------------------------------
// out = o * sigmoid(g): o, out [N][C]; g [N][g_stride] in float32 or the activations' dtype, a number for every `share`
// neighbouring columns of o (1: element by element; a head's value size: a gate per head)
// ---------------------------------------------------------------------------------------------
template <typename T, typename TG>
__global__ void sigmoid_gate_kernel(const T* __restrict__ o, const TG* __restrict__ g, long long g_stride, T* __restrict__ out,
                                    int cols, int share) {
    const int n = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    const size_t i = (size_t)n * cols + c;
    out[i] = from_f32<T>(to_f32(o[i]) / (1.0f + expf(-to_f32(g[(size_t)n * g_stride + c / share]))));
}

BLM_API int blm_sigmoid_gate(const void* o, int dtype, const void* g, int g_dtype, long long g_stride, void* out, int rows, int cols,
                             int share, cudaStream_t stream) {
    if (rows == 0 || cols == 0) return BLM_OK;
    BLM_REQUIRE(rows > 0 && rows <= 65535 && cols > 0 && share > 0, "sigmoid_gate: bad sizes");
    const int threads = 256;
    const dim3 grid((cols + threads - 1) / threads, rows);
    if (dtype == BLM_F32 && g_dtype == BLM_F32)
        sigmoid_gate_kernel<float, float><<<grid, threads, 0, stream>>>((const float*)o, (const float*)g, g_stride, (float*)out, cols, share);
    else if (dtype == BLM_BF16 && g_dtype == BLM_F32)
        sigmoid_gate_kernel<__nv_bfloat16, float><<<grid, threads, 0, stream>>>((const __nv_bfloat16*)o, (const float*)g, g_stride,
                                                                                (__nv_bfloat16*)out, cols, share);
    else if (dtype == BLM_BF16 && g_dtype == BLM_BF16)
        sigmoid_gate_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, threads, 0, stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)g,
                                                                                        g_stride, (__nv_bfloat16*)out, cols, share);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "sigmoid_gate: dtypes %d/%d", dtype, g_dtype);
    return blm_check_launch("sigmoid_gate");
}
