// Row-wise kernels around the residual stream for blocks that norm a sublayer's output before it is added:
// a scaled embedding gather, the add of a normed (and scaled) output fused with the norm that reads the stream
// next, and a bias with an optional activation.  Statistics, sums and the activation are fp32.
#include "common.cuh"

BLM_API const char* blm_stream_ops_last_error() { return g_blm_error; }

// ---------------------------------------------------------------------------------------------
// out[n, :] = table[tokens[n], :] * scale  (fp32 stream from a bf16 or fp32 table)
// ---------------------------------------------------------------------------------------------
template <typename TT>
__global__ void embed_scaled_kernel(const int* __restrict__ tokens, const TT* __restrict__ table, float* __restrict__ out,
                                    int width, int vocab, float scale) {
    const int n = blockIdx.x;
    int tok = tokens[n];
    if ((unsigned)tok >= (unsigned)vocab) tok = 0;  // ids are validated on the host; never read wild
    const TT* row = table + (size_t)tok * width;
    float* o = out + (size_t)n * width;
    for (int d = threadIdx.x; d < width; d += blockDim.x) o[d] = to_f32(row[d]) * scale;
}

BLM_API int blm_embed_scaled(const int* tokens, const void* table, int table_dtype, float* out, int n, int width, int vocab,
                             float scale, cudaStream_t stream) {
    if (n == 0) return BLM_OK;
    BLM_REQUIRE(n > 0 && width > 0 && vocab > 0, "embed_scaled: bad sizes");
    const int threads = width >= 1024 ? 256 : 128;
    if (table_dtype == BLM_BF16)
        embed_scaled_kernel<__nv_bfloat16><<<n, threads, 0, stream>>>(tokens, (const __nv_bfloat16*)table, out, width, vocab, scale);
    else if (table_dtype == BLM_F32)
        embed_scaled_kernel<float><<<n, threads, 0, stream>>>(tokens, (const float*)table, out, width, vocab, scale);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "embed_scaled: table dtype %d", table_dtype);
    return blm_check_launch("embed_scaled");
}

// ---------------------------------------------------------------------------------------------
// The sandwich step.  With d = delta (+ bias), a sublayer's raw output, or d = sa delta + sb delta2 (+ bias) for two
// mixers that ran side by side:
//     h   = resid + mult * (d / sqrt(mean(d^2) + eps_post) * post_w)          (stored unless `rows`)
//     out = h / sqrt(mean(h^2) + eps_pre) * pre_w                             (when pre_w is given)
//     out = h, converted to out's type                                        (out without pre_w: a sublayer reads the stream itself)
// delta null: h = resid.  rows given: row b of `out` comes from row rows[b]; the stream is left alone.
// ---------------------------------------------------------------------------------------------
template <typename TD, typename TA>
__global__ void sandwich_norm_kernel(float* __restrict__ resid, const TD* __restrict__ delta, const TD* __restrict__ delta2,
                                     float sa, float sb, const float* __restrict__ bias,
                                     const float* __restrict__ post_w, const float* __restrict__ pre_w, float mult,
                                     float eps_post, float eps_pre, TA* __restrict__ out, const int* __restrict__ rows,
                                     int width) {
    extern __shared__ float row_buf[];      // [width] + 33
    float* red = row_buf + width;
    const int src = rows ? rows[blockIdx.x] : blockIdx.x;
    float* r = resid + (size_t)src * width;
    float inv_d = 0.f;
    if (delta) {
        const TD* dl = delta + (size_t)src * width;
        const TD* dl2 = delta2 ? delta2 + (size_t)src * width : nullptr;
        float ss = 0.f;
        for (int d = threadIdx.x; d < width; d += blockDim.x) {
            float v = to_f32(dl[d]);
            if (dl2) v = sa * v + sb * to_f32(dl2[d]);
            if (bias) v += bias[d];
            row_buf[d] = v;
            ss += v * v;
        }
        const float total = block_sum(ss, red);
        inv_d = 1.0f / sqrtf(total / (float)width + eps_post);
    }
    float ss = 0.f;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float h = r[d];
        if (delta) {
            h += mult * (row_buf[d] * inv_d * post_w[d]);
            if (!rows) r[d] = h;
        }
        row_buf[d] = h;
        ss += h * h;
    }
    if (out == nullptr) return;
    if (pre_w == nullptr) {
        TA* o = out + (size_t)blockIdx.x * width;
        for (int d = threadIdx.x; d < width; d += blockDim.x) o[d] = from_f32<TA>(row_buf[d]);
        return;
    }
    const float total = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(total / (float)width + eps_pre);
    TA* o = out + (size_t)blockIdx.x * width;
    for (int d = threadIdx.x; d < width; d += blockDim.x) o[d] = from_f32<TA>(row_buf[d] * inv * pre_w[d]);
}

template <typename TD, typename TA>
static int launch_sandwich(float* resid, const void* delta, const void* delta2, float sa, float sb, const float* bias, const float* post_w, const float* pre_w, float mult,
                           float eps_post, float eps_pre, void* out, const int* rows, int n_rows, int width, cudaStream_t stream) {
    const size_t smem = (size_t)(width + 33) * sizeof(float);
    BLM_REQUIRE(smem <= 200 * 1024, "sandwich norm: width %d is beyond what this kernel holds in shared memory", width);
    auto k = sandwich_norm_kernel<TD, TA>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "sandwich norm: %s", cudaGetErrorString(e));
    }
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    k<<<n_rows, threads, smem, stream>>>(resid, (const TD*)delta, (const TD*)delta2, sa, sb, bias, post_w, pre_w, mult, eps_post, eps_pre, (TA*)out, rows, width);
    return blm_check_launch("sandwich_norm");
}

BLM_API int blm_sandwich_norm(float* resid, const void* delta, const void* delta2, float sa, float sb, int delta_dtype,
                              const float* bias, const float* post_w,
                              const float* pre_w, float mult, float eps_post, float eps_pre, void* out, int out_dtype,
                              const int* rows, int n_rows, int width, cudaStream_t stream) {
    if (n_rows == 0) return BLM_OK;
    BLM_REQUIRE(n_rows > 0 && width > 0, "sandwich norm: bad sizes");
    BLM_REQUIRE(delta == nullptr || post_w != nullptr, "sandwich norm: an output to add needs its norm's weight");
    BLM_REQUIRE(delta2 == nullptr || delta != nullptr, "sandwich norm: a second output without a first");
#define BLM_SW(TD, TA) return launch_sandwich<TD, TA>(resid, delta, delta2, sa, sb, bias, post_w, pre_w, mult, eps_post, eps_pre, out, rows, n_rows, width, stream)
    if (delta_dtype == BLM_F32 && out_dtype == BLM_F32) BLM_SW(float, float);
    if (delta_dtype == BLM_F32 && out_dtype == BLM_BF16) BLM_SW(float, __nv_bfloat16);
    if (delta_dtype == BLM_BF16 && out_dtype == BLM_F32) BLM_SW(__nv_bfloat16, float);
    if (delta_dtype == BLM_BF16 && out_dtype == BLM_BF16) BLM_SW(__nv_bfloat16, __nv_bfloat16);
#undef BLM_SW
    return blm_fail(BLM_BAD_ARGUMENT, "sandwich norm: dtypes %d/%d", delta_dtype, out_dtype);
}

// ---------------------------------------------------------------------------------------------
// out = act(x + bias).  kind 0: identity.  kind 1: xIELU with the two numbers params = (p, q):
//     z > 0:  softplus(p) z^2 + z / 2;     z <= 0:  (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float softplus_f(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }

template <typename TI, typename TA>
__global__ void bias_act_kernel(const TI* __restrict__ x, const float* __restrict__ bias, const float* __restrict__ params,
                                TA* __restrict__ out, int width, int kind) {
    float ap = 0.f, an = 0.f;
    if (kind == 1) {
        ap = softplus_f(params[0]);
        an = 0.5f + softplus_f(params[1]);
    }
    const size_t row = (size_t)blockIdx.y * width;       // a row a blockIdx.y: no division to find an element's bias
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < width; c += gridDim.x * blockDim.x) {
        float z = to_f32(x[row + c]);
        if (bias) z += bias[c];
        if (kind == 1) z = z > 0.f ? ap * z * z + 0.5f * z : an * (expm1f(z) - z) + 0.5f * z;
        else if (kind == 2) z = tanhf(z);
        out[row + c] = from_f32<TA>(z);
    }
}

BLM_API int blm_bias_act(const void* x, int x_dtype, const float* bias, const float* params, void* out, int out_dtype, int n,
                         int width, int kind, cudaStream_t stream) {
    if (n == 0) return BLM_OK;
    BLM_REQUIRE(n > 0 && width > 0 && (kind == 0 || kind == 1 || kind == 2), "bias_act: bad sizes or kind");
    BLM_REQUIRE(kind != 1 || params != nullptr, "bias_act: the activation needs its two numbers");
    BLM_REQUIRE(n <= 65535, "bias_act: %d rows; this kernel takes 65,535", n);
    const int threads = 256;
    dim3 grid((width + threads - 1) / threads < 64 ? (width + threads - 1) / threads : 64, n);
#define BLM_BA(TI, TA) bias_act_kernel<TI, TA><<<grid, threads, 0, stream>>>((const TI*)x, bias, params, (TA*)out, width, kind)
    if (x_dtype == BLM_F32 && out_dtype == BLM_F32) BLM_BA(float, float);
    else if (x_dtype == BLM_F32 && out_dtype == BLM_BF16) BLM_BA(float, __nv_bfloat16);
    else if (x_dtype == BLM_BF16 && out_dtype == BLM_BF16) BLM_BA(__nv_bfloat16, __nv_bfloat16);
    else if (x_dtype == BLM_BF16 && out_dtype == BLM_F32) BLM_BA(__nv_bfloat16, float);
    else return blm_fail(BLM_BAD_ARGUMENT, "bias_act: dtypes %d/%d", x_dtype, out_dtype);
#undef BLM_BA
    return blm_check_launch("bias_act");
}

// ---------------------------------------------------------------------------------------------
// out = sa a + sb b  (fp32): the sum of two mixers that ran side by side
// ---------------------------------------------------------------------------------------------
__global__ void weighted_sum_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, float sa,
                                    float sb, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        out[i] = sa * a[i] + sb * b[i];
}

BLM_API int blm_weighted_sum(const float* a, const float* b, float* out, float sa, float sb, size_t total, cudaStream_t stream) {
    if (total == 0) return BLM_OK;
    const int threads = 256;
    const size_t want = (total + threads - 1) / threads;
    const int blocks = (int)(want < 65535u * 16u ? want : 65535u * 16u);
    weighted_sum_kernel<<<blocks, threads, 0, stream>>>(a, b, out, sa, sb, total);
    return blm_check_launch("weighted_sum");
}

// ---------------------------------------------------------------------------------------------
// columns of a wider row: dst[n, col0 + d] = src[n, d] (+ delta[n, d], the sum also stored into src), converted to dst's type.
// Two calls lay the stream and another row side by side as the input of one product.  src float32 [N, D];
// delta float32 or bfloat16 [N, D] or null; dst [N, dst_stride].
// ---------------------------------------------------------------------------------------------
template <typename TD, typename TO>
__global__ void pack_cols_kernel(float* __restrict__ src, const TD* __restrict__ delta, TO* __restrict__ dst, long long dst_stride,
                                 int col0, int width) {
    const int n = blockIdx.y;
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= width) return;
    float v = src[(size_t)n * width + d];
    if (delta) {
        v += to_f32(delta[(size_t)n * width + d]);
        src[(size_t)n * width + d] = v;
    }
    dst[(size_t)n * dst_stride + col0 + d] = from_f32<TO>(v);
}

BLM_API int blm_pack_cols(float* src, const void* delta, int delta_dtype, void* dst, int dst_dtype, long long dst_stride, int col0,
                          int n_rows, int width, cudaStream_t stream) {
    if (n_rows == 0) return BLM_OK;
    BLM_REQUIRE(n_rows > 0 && n_rows <= 65535 && width > 0 && col0 >= 0 && col0 + width <= dst_stride, "pack_cols: bad sizes");
    const int threads = 256;
    dim3 grid((width + threads - 1) / threads, n_rows);
#define BLM_PC(TD, TO) pack_cols_kernel<TD, TO><<<grid, threads, 0, stream>>>(src, (const TD*)delta, (TO*)dst, dst_stride, col0, width)
    if (delta_dtype == BLM_F32 && dst_dtype == BLM_F32) BLM_PC(float, float);
    else if (delta_dtype == BLM_F32 && dst_dtype == BLM_BF16) BLM_PC(float, __nv_bfloat16);
    else if (delta_dtype == BLM_BF16 && dst_dtype == BLM_BF16) BLM_PC(__nv_bfloat16, __nv_bfloat16);
    else if (delta_dtype == BLM_BF16 && dst_dtype == BLM_F32) BLM_PC(__nv_bfloat16, float);
    else return blm_fail(BLM_BAD_ARGUMENT, "pack_cols: dtypes %d/%d", delta_dtype, dst_dtype);
#undef BLM_PC
    return blm_check_launch("pack_cols");
}

// ---------------------------------------------------------------------------------------------
// x <- cap * tanh(x / cap) in place (fp32): logits squashed into (-cap, cap)
// ---------------------------------------------------------------------------------------------
__global__ void softcap_kernel(float* __restrict__ x, float cap, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] / cap);
}

BLM_API int blm_softcap(float* x, float cap, size_t total, cudaStream_t stream) {
    if (total == 0) return BLM_OK;
    BLM_REQUIRE(cap > 0.f, "softcap: the cap must be positive");
    const int threads = 256;
    const size_t want = (total + threads - 1) / threads;
    const int blocks = (int)(want < 65535u * 16u ? want : 65535u * 16u);
    softcap_kernel<<<blocks, threads, 0, stream>>>(x, cap, total);
    return blm_check_launch("softcap");
}
