// Mixture of experts for a packed step: router, grouping of the (token, expert) pairs by expert, the experts'
// gated feed-forwards as grouped products over the pairs in that order, and the sum per token.
//
//   z = W_router h (fp32), s = sigmoid(z); a token takes its `top` experts of largest s (ties: the lower index)
//   with weight s (not renormalised).  weight_on_input: out = sum_k expert_k(s_k h); else out = sum_k s_k expert_k(h).
//   expert(x) = W_down (silu(W_gate x) * (W_up x)).
//   Options of the router: s = softmax(z) over all experts instead of the sigmoid; a correction [experts] added to the
//   scores for the choice only (the weights are the scores without it); the chosen weights divided by their sum + 1e-20.
//   A choice limited to groups: the experts form `n_groups` equal groups of neighbours, a group's mark is the sum of its
//   two largest choice scores (with the correction), and only experts of the `keep_groups` groups of largest mark (ties:
//   the lower index) can be chosen; the others' choice scores count as minus infinity.
//   Option of the experts: the clamped gated unit, g = min(W_gate x, limit), u = clamp(W_up x, -limit, limit),
//   g * sigmoid(alpha g) * (u + 1).  Or a unit without a gate, W_down act(W_up x), act the exact (erf) GELU or its tanh form.
//
// Everything runs on the device with sizes that depend on the step's token count only, so a step can be captured
// in a CUDA graph: the grids cover the worst case (every expert's share padded to a tile) and blocks beyond the
// real tiles return.
#include "common.cuh"

BLM_API const char* blm_moe_last_error() { return g_blm_error; }

// ---------------------------------------------------------------------------------------------
// router: one block per token
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ h, const float* __restrict__ router, int width, int n_experts, int top,
                                 int* __restrict__ ids, float* __restrict__ weights, int softmax, const float* __restrict__ correction,
                                 int renorm, int n_groups, int keep_groups) {
    extern __shared__ __align__(16) float smem[];
    float* x = smem;                     // [width]
    float* score = smem + width;         // [n_experts]: what a chosen expert is weighted by
    float* choice = score + n_experts;   // [n_experts]: what the choice looks at (the score, plus the correction)
    float* mark = choice + n_experts;    // [n_groups]: the groups' marks
    const int n = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int d = threadIdx.x; d < width; d += blockDim.x) x[d] = to_f32(h[(size_t)n * width + d]);
    __syncthreads();
    for (int e = warp; e < n_experts; e += n_warps) {
        const float* w = router + (size_t)e * width;
        float z = 0.f;
        if ((width & 127) == 0) {            // four loads of 16 bytes on their way at once, four sums: the loop waits for memory, not for itself
            const float4* w4 = reinterpret_cast<const float4*>(w);
            const float4* x4 = reinterpret_cast<const float4*>(x);
            float z0 = 0.f, z1 = 0.f, z2 = 0.f, z3 = 0.f;
#pragma unroll 8
            for (int d = lane; d < width / 4; d += 32) {
                const float4 a = __ldg(w4 + d), c = x4[d];
                z0 = fmaf(a.x, c.x, z0); z1 = fmaf(a.y, c.y, z1); z2 = fmaf(a.z, c.z, z2); z3 = fmaf(a.w, c.w, z3);
            }
            z = (z0 + z1) + (z2 + z3);
        } else {
            for (int d = lane; d < width; d += 32) z = fmaf(w[d], x[d], z);
        }
        z = warp_sum(z);
        // (a row of no sequence may hold anything, a NaN too: its score is 0, so that it still names experts that exist)
        if (lane == 0) score[e] = softmax ? (z == z ? z : 0.f) : (z == z ? 1.0f / (1.0f + expf(-z)) : 0.f);
    }
    __syncthreads();
    if (warp == 0) {
        if (softmax) {
            float m = -INFINITY;
            for (int e = lane; e < n_experts; e += 32) m = fmaxf(m, score[e]);
            m = warp_max(m);
            float sum = 0.f;
            for (int e = lane; e < n_experts; e += 32) {
                const float p = expf(score[e] - m);
                score[e] = p;
                sum += p;
            }
            sum = warp_sum(sum);
            for (int e = lane; e < n_experts; e += 32) score[e] = score[e] / sum;
        }
        for (int e = lane; e < n_experts; e += 32) choice[e] = correction ? score[e] + correction[e] : score[e];
        __syncwarp();
        if (n_groups > 1 && keep_groups < n_groups) {
            const int per = n_experts / n_groups;
            for (int g = lane; g < n_groups; g += 32) {          // a group's mark: its two largest choice scores
                float a = -INFINITY, b = -INFINITY;
                for (int e = g * per; e < (g + 1) * per; ++e) {
                    const float c = choice[e];
                    if (c > a) { b = a; a = c; } else if (c > b) b = c;
                }
                mark[g] = per > 1 ? a + b : a;
            }
            __syncwarp();
            for (int g = lane; g < n_groups; g += 32) {          // kept when fewer than keep_groups groups come before it
                const float mine = mark[g];
                int ahead = 0;
                for (int o = 0; o < n_groups; ++o) ahead += (mark[o] > mine || (mark[o] == mine && o < g)) ? 1 : 0;
                if (ahead >= keep_groups)
                    for (int e = g * per; e < (g + 1) * per; ++e) choice[e] = -INFINITY;
            }
            __syncwarp();
        }
        float total = 0.f;
        for (int k = 0; k < top; ++k) {
            float best = -INFINITY;
            int arg = 0x7fffffff;
            for (int e = lane; e < n_experts; e += 32) {
                const float s = choice[e];
                if (s > best) { best = s; arg = e; }     // ascending e per lane: the lower index stays on a tie
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
                if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
            }
            if (arg == 0x7fffffff) arg = k;              // (scores that compare with nothing: still an expert that exists)
            const float wgt = score[arg];
            total += wgt;
            if (lane == 0) {
                ids[(size_t)n * top + k] = arg;
                weights[(size_t)n * top + k] = wgt;
                choice[arg] = -INFINITY;                 // taken
            }
            __syncwarp();
        }
        if (renorm)
            for (int k = lane; k < top; k += 32) weights[(size_t)n * top + k] = weights[(size_t)n * top + k] / (total + 1e-20f);
    }
}

BLM_API int blm_moe_route(const void* h, int dtype, const float* router, int n_tokens, int width, int n_experts, int top, int* ids,
                          float* weights, int softmax, const float* correction, int renorm, int n_groups, int keep_groups,
                          cudaStream_t stream) {
    // n_groups <= 1: the choice is among all experts
    if (n_tokens == 0) return BLM_OK;
    BLM_REQUIRE(n_tokens > 0 && width > 0 && n_experts > 0 && top > 0 && top <= n_experts, "moe_route: bad sizes");
    if (n_groups < 1) n_groups = 1;
    BLM_REQUIRE(n_experts % n_groups == 0 && keep_groups >= 1 && keep_groups <= n_groups &&
                (long long)keep_groups * (n_experts / n_groups) >= top,
                "moe_route: %d experts in %d groups of which %d are kept, for %d chosen", n_experts, n_groups, keep_groups, top);
    const size_t smem = ((size_t)width + 2 * n_experts + n_groups) * sizeof(float);
    BLM_REQUIRE(smem <= 48 * 1024, "moe_route: width %d and %d experts need %zu bytes of shared memory", width, n_experts, smem);
    // a warp an expert where the experts are few (the warps' dot products wait for memory side by side), sixteen warps at most
    const int threads = n_experts <= 4 ? 128 : (n_experts >= 16 ? 512 : 32 * n_experts);
    if (dtype == BLM_F32)
        moe_route_kernel<float><<<n_tokens, threads, smem, stream>>>((const float*)h, router, width, n_experts, top, ids, weights, softmax,
                                                                 correction, renorm, n_groups, keep_groups);
    else if (dtype == BLM_BF16)
        moe_route_kernel<__nv_bfloat16><<<n_tokens, threads, smem, stream>>>((const __nv_bfloat16*)h, router, width, n_experts, top, ids,
                                                                         weights, softmax, correction, renorm, n_groups, keep_groups);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "moe_route: dtype %d", dtype);
    return blm_check_launch("moe_route");
}

// ---------------------------------------------------------------------------------------------
// grouping: offsets[e] .. offsets[e + 1] are the places of expert e's pairs; order[place] = pair (token * top + k);
// place_of[pair] = place.  One block.  The order inside an expert's share is whatever the atomics give: every
// pair's row is computed on its own, so no result depends on it.
// ---------------------------------------------------------------------------------------------
__global__ void moe_group_kernel(const int* __restrict__ ids, int n_pairs, int n_experts, int* __restrict__ offsets,
                                 int* __restrict__ order, int* __restrict__ place_of) {
    extern __shared__ int counts[];      // [n_experts] counts, then [n_experts] cursors
    int* cursor = counts + n_experts;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int a = threadIdx.x; a < n_pairs; a += blockDim.x) atomicAdd(&counts[min(max(ids[a], 0), n_experts - 1)], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < n_experts; ++e) {
            offsets[e] = run;
            cursor[e] = run;
            run += counts[e];
        }
        offsets[n_experts] = run;
    }
    __syncthreads();
    for (int a = threadIdx.x; a < n_pairs; a += blockDim.x) {
        const int place = atomicAdd(&cursor[min(max(ids[a], 0), n_experts - 1)], 1);
        order[place] = a;
        place_of[a] = place;
    }
}

BLM_API int blm_moe_group(const int* ids, int n_pairs, int n_experts, int* offsets, int* order, int* place_of, cudaStream_t stream) {
    if (n_pairs == 0) return BLM_OK;
    BLM_REQUIRE(n_pairs > 0 && n_experts > 0 && n_experts <= 4096, "moe_group: bad sizes");
    moe_group_kernel<<<1, 1024, 2 * (size_t)n_experts * sizeof(int), stream>>>(ids, n_pairs, n_experts, offsets, order, place_of);
    return blm_check_launch("moe_group");
}

// ---------------------------------------------------------------------------------------------
// grouped products on the CUDA cores (fp32 sums): tiles of kBM places x kBN outputs, the reduction in slices of
// kBK.  A block finds the expert and the places of its tile from the offsets; blocks beyond the last tile return.
// ---------------------------------------------------------------------------------------------
constexpr int kBM = 32, kBN = 32, kBK = 32;

__device__ __forceinline__ bool moe_find_tile(const int* __restrict__ offsets, int n_experts, int tile, int* expert, int* first, int* last,
                                              int tile_rows = kBM) {
    __shared__ int found[3];
    if (threadIdx.x == 0) {
        int t = tile, e = 0;
        found[0] = -1;
        for (; e < n_experts; ++e) {
            const int begin = offsets[e], end = offsets[e + 1];
            const int tiles = (end - begin + tile_rows - 1) / tile_rows;
            if (t < tiles) {
                found[0] = e;
                found[1] = begin + t * tile_rows;
                found[2] = end;
                break;
            }
            t -= tiles;
        }
    }
    __syncthreads();
    *expert = found[0];
    *first = found[1];
    *last = found[2];
    return found[0] >= 0;
}

// x rounded as the activations' dtype rounds it: the input of a product in that dtype
template <typename T> __device__ __forceinline__ float as_input(float v) { return to_f32(from_f32<T>(v)); }

// The unit of an expert.  plain 0, the gated units: limit <= 0: silu(g) * u; limit > 0, the clamped unit: g = min(g, limit),
// u = clamp(u, -limit, limit), g * sigmoid(alpha g) * (u + 1).  plain 1 and 2, the units without a gate (the weight then
// holds the up rows only, and u is not computed): the exact GELU, g (1 + erf(g / sqrt 2)) / 2, and its tanh form.
struct GluAct {
    float limit, alpha;
    int plain;
};
__device__ __forceinline__ float glu_act(float g, float u, GluAct a) {
    if (a.plain == 1) return 0.5f * g * (1.0f + erff(g * 0.70710678118654752f));
    if (a.plain == 2) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    if (a.limit <= 0.f) return g / (1.0f + expf(-g)) * u;
    g = fminf(g, a.limit);
    u = fminf(fmaxf(u, -a.limit), a.limit);
    return g / (1.0f + expf(-a.alpha * g)) * (u + 1.0f);
}

// act[place, c] = silu(x . Wgate[e, c]) * (x . Wup[e, c]),  x = the pair's token row of h (times the pair's weight when
// `scale_input`).  w_gu: [experts, 2 ff, width], an expert's gate rows followed by its up rows.
template <typename T>
__global__ void moe_gate_up_kernel(const T* __restrict__ h, const float* __restrict__ weights, const int* __restrict__ order,
                                   const int* __restrict__ offsets, const T* __restrict__ w_gu, T* __restrict__ act, int width, int ff,
                                   int n_experts, int top, int scale_input, GluAct glu) {
    __shared__ float xs[kBM][kBK + 1], gs[kBN][kBK + 1], us[kBN][kBK + 1];
    __shared__ int token_of[kBM];
    __shared__ float scale_of[kBM];
    int e, first, last;
    if (!moe_find_tile(offsets, n_experts, blockIdx.x, &e, &first, &last)) return;
    const int c0 = blockIdx.y * kBN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;       // 16 x 16 threads, 2 places x 2 outputs each
    if (threadIdx.x < kBM) {
        const int place = first + threadIdx.x;
        int tok = -1;
        float sc = 1.f;
        if (place < last) {
            const int pair = order[place];
            tok = pair / top;
            if (scale_input) sc = weights[pair];
        }
        token_of[threadIdx.x] = tok;
        scale_of[threadIdx.x] = sc;
    }
    __syncthreads();
    const bool gated = glu.plain == 0;
    const T* wg = w_gu + (size_t)e * (gated ? 2 : 1) * ff * width;
    const T* wu = wg + (size_t)ff * width;
    float ag[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, au[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    for (int k0 = 0; k0 < width; k0 += kBK) {
        for (int idx = threadIdx.x; idx < kBM * kBK; idx += blockDim.x) {
            const int r = idx / kBK, kk = idx % kBK, k = k0 + kk;
            const int tok = token_of[r];
            float v = 0.f;
            if (tok >= 0 && k < width) {
                v = to_f32(h[(size_t)tok * width + k]);
                if (scale_input) v = as_input<T>(scale_of[r] * v);
            }
            xs[r][kk] = v;
        }
        for (int idx = threadIdx.x; idx < kBN * kBK; idx += blockDim.x) {
            const int r = idx / kBK, kk = idx % kBK, k = k0 + kk, c = c0 + r;
            const bool in = c < ff && k < width;
            gs[r][kk] = in ? to_f32(wg[(size_t)c * width + k]) : 0.f;
            us[r][kk] = in && gated ? to_f32(wu[(size_t)c * width + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kBK; ++kk) {
            const float x0 = xs[ty][kk], x1 = xs[ty + 16][kk];
            const float g0 = gs[tx][kk], g1 = gs[tx + 16][kk], u0 = us[tx][kk], u1 = us[tx + 16][kk];
            ag[0][0] = fmaf(x0, g0, ag[0][0]); ag[0][1] = fmaf(x0, g1, ag[0][1]);
            ag[1][0] = fmaf(x1, g0, ag[1][0]); ag[1][1] = fmaf(x1, g1, ag[1][1]);
            au[0][0] = fmaf(x0, u0, au[0][0]); au[0][1] = fmaf(x0, u1, au[0][1]);
            au[1][0] = fmaf(x1, u0, au[1][0]); au[1][1] = fmaf(x1, u1, au[1][1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int place = first + ty + 16 * i, c = c0 + tx + 16 * j;
            if (place < last && c < ff) {
                act[(size_t)place * ff + c] = from_f32<T>(glu_act(ag[i][j], au[i][j], glu));
            }
        }
}

// y[place, c] = act[place] . Wdown[e, c]   (fp32 out).  w_down: [experts, width, ff].
template <typename T>
__global__ void moe_down_kernel(const T* __restrict__ act, const int* __restrict__ offsets, const T* __restrict__ w_down,
                                float* __restrict__ y, int width, int ff, int n_experts) {
    __shared__ float xs[kBM][kBK + 1], ws[kBN][kBK + 1];
    int e, first, last;
    if (!moe_find_tile(offsets, n_experts, blockIdx.x, &e, &first, &last)) return;
    const int c0 = blockIdx.y * kBN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const T* wd = w_down + (size_t)e * width * ff;
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    for (int k0 = 0; k0 < ff; k0 += kBK) {
        for (int idx = threadIdx.x; idx < kBM * kBK; idx += blockDim.x) {
            const int r = idx / kBK, kk = idx % kBK, k = k0 + kk, place = first + r;
            xs[r][kk] = (place < last && k < ff) ? to_f32(act[(size_t)place * ff + k]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < kBN * kBK; idx += blockDim.x) {
            const int r = idx / kBK, kk = idx % kBK, k = k0 + kk, c = c0 + r;
            ws[r][kk] = (c < width && k < ff) ? to_f32(wd[(size_t)c * ff + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kBK; ++kk) {
            const float x0 = xs[ty][kk], x1 = xs[ty + 16][kk], w0 = ws[tx][kk], w1 = ws[tx + 16][kk];
            acc[0][0] = fmaf(x0, w0, acc[0][0]); acc[0][1] = fmaf(x0, w1, acc[0][1]);
            acc[1][0] = fmaf(x1, w0, acc[1][0]); acc[1][1] = fmaf(x1, w1, acc[1][1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int place = first + ty + 16 * i, c = c0 + tx + 16 * j;
            if (place < last && c < width) y[(size_t)place * width + c] = acc[i][j];
        }
}

// ---------------------------------------------------------------------------------------------
// The same grouped products on the tensor cores (bfloat16, mma.sync m16n8k16 with fp32 sums, operands fetched with
// ldmatrix): tiles of 64 places x 64 outputs, the reduction in slices of 64 that come through cp.async into two
// buffers in turn; four warps, each 16 places of the tile.  Width and inner size are multiples of 8 (16-byte copies).
// A weight on the expert's input is applied to both products' sums instead, W (s x) = s (W x), in fp32.
// ---------------------------------------------------------------------------------------------
#ifndef BLM_MOE_TK
#define BLM_MOE_TK 64
#endif
constexpr int kTM = 64, kTN = 64, kTK = BLM_MOE_TK, kTStride = kTK + 8;     // rows 16 bytes apart modulo 128: ldmatrix reads eight at once
constexpr int kTile = kTM * kTStride;                               // elements of one staged operand

__device__ __forceinline__ void moe_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// `a`: a shared-memory address (32 bits, from __cvta_generic_to_shared once per operand: the offsets of a tile are constants)
__device__ __forceinline__ void moe_ldsm_x4(uint32_t (&r)[4], unsigned a) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void moe_cp16(__nv_bfloat16* dst, const __nv_bfloat16* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;                  // zeros where nothing is to be read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void moe_cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void moe_cp_wait_all_but() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
// Slices of the reduction in shared memory at once: one worked on, the others on their way.  Measured with 8 experts of
// 6,144 x 2,048 (10,752 x 4,096) without gates, 2 chosen: two slices of 64 lanes 198 / 215 / 1,110 us for 8 / 64 / 2,048 tokens
// (450 / 574 / 3,664); three slices 196 / 221 / 1,144 (453 / 535 / 3,780); four 196 / 219 / 1,213 (554 / 621 / 4,007); two
// slices of 128 lanes (-DBLM_MOE_TK=128) 166 / 208 / 1,157 (363 / 563 / 3,811); of 256 lanes 230 / 277 / 1,963.  So two
// slices of 64 it stays: more copies in flight do not help, longer pieces of a weight row help the fewest tokens only.
#ifndef BLM_MOE_STAGES
#define BLM_MOE_STAGES 2
#endif
constexpr int kMoeStages = BLM_MOE_STAGES;

// rows [c0, c0 + 64) x lanes [k0, k0 + 64) of a weight [n_rows, n_cols] into ws[64][kTStride]; zeros outside
__device__ __forceinline__ void moe_stage_weight(__nv_bfloat16* ws, const __nv_bfloat16* __restrict__ w, int n_rows, int n_cols, int c0, int k0) {
    for (int idx = threadIdx.x; idx < kTN * (kTK / 8); idx += blockDim.x) {
        const int r = idx / (kTK / 8), kk = (idx % (kTK / 8)) * 8;
        const bool in = c0 + r < n_rows && k0 + kk < n_cols;
        moe_cp16(ws + r * kTStride + kk, in ? w + (size_t)(c0 + r) * n_cols + k0 + kk : w, in);
    }
}

// 16 places x 64 outputs of one warp: acc[j] += x (16 x 64 slice) . w (64 outputs x 64 slice)
__device__ __forceinline__ void moe_warp_product(float (&acc)[8][4], unsigned xa, unsigned wb) {
#pragma unroll
    for (int kk = 0; kk < kTK; kk += 16) {
        uint32_t a[4], b[4];
        moe_ldsm_x4(a, xa + kk * 2);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            moe_ldsm_x4(b, wb + (16 * jj * kTStride + kk) * 2);
            moe_mma(acc[2 * jj], a, b[0], b[1]);
            moe_mma(acc[2 * jj + 1], a, b[2], b[3]);
        }
    }
}

// the gate's and the up projection's sums of one slice in one pass over the tokens' operand
__device__ __forceinline__ void moe_warp_product2(float (&g)[8][4], float (&u)[8][4], unsigned xa, unsigned gb, unsigned ub) {
#pragma unroll
    for (int kk = 0; kk < kTK; kk += 16) {
        uint32_t a[4], b[4];
        moe_ldsm_x4(a, xa + kk * 2);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            moe_ldsm_x4(b, gb + (16 * jj * kTStride + kk) * 2);
            moe_mma(g[2 * jj], a, b[0], b[1]);
            moe_mma(g[2 * jj + 1], a, b[2], b[3]);
            moe_ldsm_x4(b, ub + (16 * jj * kTStride + kk) * 2);
            moe_mma(u[2 * jj], a, b[0], b[1]);
            moe_mma(u[2 * jj + 1], a, b[2], b[3]);
        }
    }
}

template <bool kGated>
__global__ void __launch_bounds__(128) moe_gate_up_tc_kernel(const __nv_bfloat16* __restrict__ h, const float* __restrict__ weights,
                                                             const int* __restrict__ order, const int* __restrict__ offsets,
                                                             const __nv_bfloat16* __restrict__ w_gu, __nv_bfloat16* __restrict__ act,
                                                             int width, int ff, int n_experts, int top, int scale_input, GluAct glu) {
    extern __shared__ __align__(16) unsigned char moe_smem[];
    __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(moe_smem);      // kMoeStages x (x, gate, up); without a gate: (x, up)
    constexpr int kOperands = kGated ? 3 : 2;
    __shared__ int token_of[kTM];
    __shared__ float scale_of[kTM];
    int e, first, last;
    if (!moe_find_tile(offsets, n_experts, blockIdx.x, &e, &first, &last, kTM)) return;
    const int c0 = blockIdx.y * kTN;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, quad = lane >> 2, pair = (lane & 3) * 2;
    const int lrow = lane & 7, lmat = lane >> 3;
    if (threadIdx.x < kTM) {
        const int place = first + threadIdx.x;
        int tok = -1;
        float sc = 1.f;
        if (place < last) {
            const int p = order[place];
            tok = p / top;
            if (scale_input) sc = weights[p];
        }
        token_of[threadIdx.x] = tok;
        scale_of[threadIdx.x] = sc;
    }
    __syncthreads();
    const __nv_bfloat16* wg = w_gu + (size_t)e * (kGated ? 2 : 1) * ff * width;
    const __nv_bfloat16* wu = wg + (size_t)ff * width;
    auto stage_slice = [&](int buf, int k0) {
        __nv_bfloat16* xs = stage + buf * kOperands * kTile;
        for (int idx = threadIdx.x; idx < kTM * (kTK / 8); idx += blockDim.x) {
            const int r = idx / (kTK / 8), kk = (idx % (kTK / 8)) * 8;
            const int tok = token_of[r];
            const bool in = tok >= 0 && k0 + kk < width;
            moe_cp16(xs + r * kTStride + kk, in ? h + (size_t)tok * width + k0 + kk : h, in);
        }
        moe_stage_weight(xs + kTile, wg, ff, width, c0, k0);
        if (kGated) moe_stage_weight(xs + 2 * kTile, wu, ff, width, c0, k0);
    };
    float g[8][4], u[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j][0] = g[j][1] = g[j][2] = g[j][3] = u[j][0] = u[j][1] = u[j][2] = u[j][3] = 0.f;
    const int a_off = (warp * 16 + lrow + (lmat & 1) * 8) * kTStride + (lmat >> 1) * 8;
    const int b_off = (lrow + (lmat >> 1) * 8) * kTStride + (lmat & 1) * 8;
    const unsigned stage_at = (unsigned)__cvta_generic_to_shared(stage);
    const int n_slices = (width + kTK - 1) / kTK;
#pragma unroll
    for (int ahead = 0; ahead < kMoeStages - 1; ++ahead) {
        if (ahead < n_slices) stage_slice(ahead, ahead * kTK);
        moe_cp_commit();
    }
    for (int it = 0; it < n_slices; ++it) {
        const int buf = it % kMoeStages;
        if (it + kMoeStages - 1 < n_slices) stage_slice((it + kMoeStages - 1) % kMoeStages, (it + kMoeStages - 1) * kTK);   // where the slice before this one lay
        moe_cp_commit();
        moe_cp_wait_all_but<kMoeStages - 1>();
        __syncthreads();
        const unsigned xs = stage_at + buf * kOperands * kTile * 2;
        if (kGated) moe_warp_product2(g, u, xs + a_off * 2, xs + (kTile + b_off) * 2, xs + (2 * kTile + b_off) * 2);
        else moe_warp_product(g, xs + a_off * 2, xs + (kTile + b_off) * 2);
        __syncthreads();
    }
    const int r0 = warp * 16 + quad, r1 = r0 + 8;
    const int p0 = first + r0, p1 = first + r1;
    const float s0 = scale_of[r0], s1 = scale_of[r1];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int c = c0 + 8 * j + pair;
        if (c < ff) {                                   // ff is even: c + 1 < ff as well
            if (p0 < last) {
                const float x = s0 * g[j][0], y = s0 * g[j][1];
                *reinterpret_cast<__nv_bfloat162*>(act + (size_t)p0 * ff + c) =
                    __floats2bfloat162_rn(glu_act(x, s0 * u[j][0], glu), glu_act(y, s0 * u[j][1], glu));
            }
            if (p1 < last) {
                const float x = s1 * g[j][2], y = s1 * g[j][3];
                *reinterpret_cast<__nv_bfloat162*>(act + (size_t)p1 * ff + c) =
                    __floats2bfloat162_rn(glu_act(x, s1 * u[j][2], glu), glu_act(y, s1 * u[j][3], glu));
            }
        }
    }
}

__global__ void __launch_bounds__(128) moe_down_tc_kernel(const __nv_bfloat16* __restrict__ act, const int* __restrict__ offsets,
                                                          const __nv_bfloat16* __restrict__ w_down, float* __restrict__ y, int width, int ff,
                                                          int n_experts) {
    extern __shared__ __align__(16) unsigned char moe_smem[];
    __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(moe_smem);      // kMoeStages x (x, weight)
    int e, first, last;
    if (!moe_find_tile(offsets, n_experts, blockIdx.x, &e, &first, &last, kTM)) return;
    const int c0 = blockIdx.y * kTN;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, quad = lane >> 2, pair = (lane & 3) * 2;
    const int lrow = lane & 7, lmat = lane >> 3;
    const __nv_bfloat16* wd = w_down + (size_t)e * width * ff;
    auto stage_slice = [&](int buf, int k0) {
        __nv_bfloat16* xs = stage + buf * 2 * kTile;
        for (int idx = threadIdx.x; idx < kTM * (kTK / 8); idx += blockDim.x) {
            const int r = idx / (kTK / 8), kk = (idx % (kTK / 8)) * 8;
            const bool in = first + r < last && k0 + kk < ff;
            moe_cp16(xs + r * kTStride + kk, in ? act + (size_t)(first + r) * ff + k0 + kk : act, in);
        }
        moe_stage_weight(xs + kTile, wd, width, ff, c0, k0);
    };
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    const int a_off = (warp * 16 + lrow + (lmat & 1) * 8) * kTStride + (lmat >> 1) * 8;
    const int b_off = (lrow + (lmat >> 1) * 8) * kTStride + (lmat & 1) * 8;
    const unsigned stage_at = (unsigned)__cvta_generic_to_shared(stage);
    const int n_slices = (ff + kTK - 1) / kTK;
#pragma unroll
    for (int ahead = 0; ahead < kMoeStages - 1; ++ahead) {
        if (ahead < n_slices) stage_slice(ahead, ahead * kTK);
        moe_cp_commit();
    }
    for (int it = 0; it < n_slices; ++it) {
        const int buf = it % kMoeStages;
        if (it + kMoeStages - 1 < n_slices) stage_slice((it + kMoeStages - 1) % kMoeStages, (it + kMoeStages - 1) * kTK);
        moe_cp_commit();
        moe_cp_wait_all_but<kMoeStages - 1>();
        __syncthreads();
        const unsigned xs = stage_at + buf * 2 * kTile * 2;
        moe_warp_product(acc, xs + a_off * 2, xs + (kTile + b_off) * 2);
        __syncthreads();
    }
    const int p0 = first + warp * 16 + quad, p1 = p0 + 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int c = c0 + 8 * j + pair;
        if (c < width) {                                // width is even
            if (p0 < last) *reinterpret_cast<float2*>(y + (size_t)p0 * width + c) = make_float2(acc[j][0], acc[j][1]);
            if (p1 < last) *reinterpret_cast<float2*>(y + (size_t)p1 * width + c) = make_float2(acc[j][2], acc[j][3]);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The same products for steps that bring an expert a few tokens only (single-token steps of a batch): tiles of 16 places x
// 64 outputs, the four warps of a block 16 outputs each, the reduction in slices of 128 lanes (longer pieces of a weight
// row a copy).  With tiles of 64 places three warps in four multiplied rows of zeros, and the blocks were bound by the
// instructions they issued, not by the weights they stream.  The second product has few output tiles (width / 64 a
// tile of places), so its reduction is cut over gridDim.z blocks, each of which leaves its share of the sums in a plane of
// its own ([splits][places][width]); the kernel that sums a token's experts adds the planes in order.
// ---------------------------------------------------------------------------------------------
constexpr int kSM = 16, kSN = 64, kSK = 128, kSStride = kSK + 8;
constexpr int kSTileX = kSM * kSStride, kSTileW = kSN * kSStride;
#ifndef BLM_MOE_SKINNY_PAIRS
#define BLM_MOE_SKINNY_PAIRS 32      // up to this many (token, expert) pairs an expert on average the skinny kernels run
#endif

__device__ __forceinline__ void moe_stage_weight_skinny(__nv_bfloat16* ws, const __nv_bfloat16* __restrict__ w, int n_rows, int n_cols, int c0,
                                                        int k0, int k_end) {
    for (int idx = threadIdx.x; idx < kSN * (kSK / 8); idx += blockDim.x) {
        const int r = idx / (kSK / 8), kk = (idx % (kSK / 8)) * 8;
        const bool in = c0 + r < n_rows && k0 + kk < k_end;
        moe_cp16(ws + r * kSStride + kk, in ? w + (size_t)(c0 + r) * n_cols + k0 + kk : w, in);
    }
}

template <bool kGated>
__global__ void __launch_bounds__(128) moe_up_skinny_kernel(const __nv_bfloat16* __restrict__ h, const float* __restrict__ weights,
                                                            const int* __restrict__ order, const int* __restrict__ offsets,
                                                            const __nv_bfloat16* __restrict__ w_gu, __nv_bfloat16* __restrict__ act,
                                                            int width, int ff, int n_experts, int top, int scale_input, GluAct glu) {
    extern __shared__ __align__(16) unsigned char moe_smem[];
    __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(moe_smem);      // 2 x (x, gate, up); without a gate: (x, up)
    constexpr int kStage = kSTileX + (kGated ? 2 : 1) * kSTileW;
    __shared__ int token_of[kSM];
    __shared__ float scale_of[kSM];
    int e, first, last;
    if (!moe_find_tile(offsets, n_experts, blockIdx.x, &e, &first, &last, kSM)) return;
    const int c0 = blockIdx.y * kSN;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, quad = lane >> 2, pair = (lane & 3) * 2;
    const int lrow = lane & 7, lmat = lane >> 3;
    if (threadIdx.x < kSM) {
        const int place = first + threadIdx.x;
        int tok = -1;
        float sc = 1.f;
        if (place < last) {
            const int p = order[place];
            tok = p / top;
            if (scale_input) sc = weights[p];
        }
        token_of[threadIdx.x] = tok;
        scale_of[threadIdx.x] = sc;
    }
    __syncthreads();
    const __nv_bfloat16* wg = w_gu + (size_t)e * (kGated ? 2 : 1) * ff * width;
    const __nv_bfloat16* wu = wg + (size_t)ff * width;
    auto stage_slice = [&](int buf, int k0) {
        __nv_bfloat16* xs = stage + buf * kStage;
        for (int idx = threadIdx.x; idx < kSM * (kSK / 8); idx += blockDim.x) {
            const int r = idx / (kSK / 8), kk = (idx % (kSK / 8)) * 8;
            const int tok = token_of[r];
            const bool in = tok >= 0 && k0 + kk < width;
            moe_cp16(xs + r * kSStride + kk, in ? h + (size_t)tok * width + k0 + kk : h, in);
        }
        moe_stage_weight_skinny(xs + kSTileX, wg, ff, width, c0, k0, width);
        if (kGated) moe_stage_weight_skinny(xs + kSTileX + kSTileW, wu, ff, width, c0, k0, width);
    };
    float g[2][4], u[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) g[j][0] = g[j][1] = g[j][2] = g[j][3] = u[j][0] = u[j][1] = u[j][2] = u[j][3] = 0.f;
    const int a_off = (lrow + (lmat & 1) * 8) * kSStride + (lmat >> 1) * 8;
    const int b_off = (warp * 16 + lrow + (lmat >> 1) * 8) * kSStride + (lmat & 1) * 8;
    const unsigned stage_at = (unsigned)__cvta_generic_to_shared(stage);
    stage_slice(0, 0);
    moe_cp_commit();
    const int n_slices = (width + kSK - 1) / kSK;
    for (int it = 0; it < n_slices; ++it) {
        const int buf = it & 1;
        if (it + 1 < n_slices) stage_slice(buf ^ 1, (it + 1) * kSK);
        moe_cp_commit();
        moe_cp_wait_all_but<1>();
        __syncthreads();
        const unsigned xs = stage_at + buf * kStage * 2;
#pragma unroll
        for (int kk = 0; kk < kSK; kk += 16) {
            uint32_t a[4], b[4];
            moe_ldsm_x4(a, xs + (a_off + kk) * 2);
            moe_ldsm_x4(b, xs + (kSTileX + b_off + kk) * 2);
            moe_mma(g[0], a, b[0], b[1]);
            moe_mma(g[1], a, b[2], b[3]);
            if (kGated) {
                moe_ldsm_x4(b, xs + (kSTileX + kSTileW + b_off + kk) * 2);
                moe_mma(u[0], a, b[0], b[1]);
                moe_mma(u[1], a, b[2], b[3]);
            }
        }
        __syncthreads();
    }
    const int p0 = first + quad, p1 = p0 + 8;
    const float s0 = scale_of[quad], s1 = scale_of[quad + 8];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int c = c0 + warp * 16 + 8 * j + pair;
        if (c < ff) {                                   // ff is even: c + 1 < ff as well
            if (p0 < last)
                *reinterpret_cast<__nv_bfloat162*>(act + (size_t)p0 * ff + c) =
                    __floats2bfloat162_rn(glu_act(s0 * g[j][0], s0 * u[j][0], glu), glu_act(s0 * g[j][1], s0 * u[j][1], glu));
            if (p1 < last)
                *reinterpret_cast<__nv_bfloat162*>(act + (size_t)p1 * ff + c) =
                    __floats2bfloat162_rn(glu_act(s1 * g[j][2], s1 * u[j][2], glu), glu_act(s1 * g[j][3], s1 * u[j][3], glu));
        }
    }
}

// y[z][place, c] = sum over the z-th share of k of act[place, k] Wdown[e, c, k]
__global__ void __launch_bounds__(128) moe_down_skinny_kernel(const __nv_bfloat16* __restrict__ act, const int* __restrict__ offsets,
                                                              const __nv_bfloat16* __restrict__ w_down, float* __restrict__ y, int width, int ff,
                                                              int n_experts, long long plane) {
    extern __shared__ __align__(16) unsigned char moe_smem[];
    __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(moe_smem);      // 2 x (x, weight)
    constexpr int kStage = kSTileX + kSTileW;
    int e, first, last;
    if (!moe_find_tile(offsets, n_experts, blockIdx.x, &e, &first, &last, kSM)) return;
    const int c0 = blockIdx.y * kSN;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, quad = lane >> 2, pair = (lane & 3) * 2;
    const int lrow = lane & 7, lmat = lane >> 3;
    const int slices_all = (ff + kSK - 1) / kSK, per = (slices_all + (int)gridDim.z - 1) / (int)gridDim.z;
    const int k_begin = min(ff, (int)blockIdx.z * per * kSK), k_end = min(ff, ((int)blockIdx.z + 1) * per * kSK);
    const __nv_bfloat16* wd = w_down + (size_t)e * width * ff;
    auto stage_slice = [&](int buf, int k0) {
        __nv_bfloat16* xs = stage + buf * kStage;
        for (int idx = threadIdx.x; idx < kSM * (kSK / 8); idx += blockDim.x) {
            const int r = idx / (kSK / 8), kk = (idx % (kSK / 8)) * 8;
            const bool in = first + r < last && k0 + kk < k_end;
            moe_cp16(xs + r * kSStride + kk, in ? act + (size_t)(first + r) * ff + k0 + kk : act, in);
        }
        moe_stage_weight_skinny(xs + kSTileX, wd, width, ff, c0, k0, k_end);
    };
    float acc[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    const int a_off = (lrow + (lmat & 1) * 8) * kSStride + (lmat >> 1) * 8;
    const int b_off = (warp * 16 + lrow + (lmat >> 1) * 8) * kSStride + (lmat & 1) * 8;
    const unsigned stage_at = (unsigned)__cvta_generic_to_shared(stage);
    const int n_slices = (k_end - k_begin + kSK - 1) / kSK;
    if (n_slices > 0) stage_slice(0, k_begin);
    moe_cp_commit();
    for (int it = 0; it < n_slices; ++it) {
        const int buf = it & 1;
        if (it + 1 < n_slices) stage_slice(buf ^ 1, k_begin + (it + 1) * kSK);
        moe_cp_commit();
        moe_cp_wait_all_but<1>();
        __syncthreads();
        const unsigned xs = stage_at + buf * kStage * 2;
#pragma unroll
        for (int kk = 0; kk < kSK; kk += 16) {
            uint32_t a[4], b[4];
            moe_ldsm_x4(a, xs + (a_off + kk) * 2);
            moe_ldsm_x4(b, xs + (kSTileX + b_off + kk) * 2);
            moe_mma(acc[0], a, b[0], b[1]);
            moe_mma(acc[1], a, b[2], b[3]);
        }
        __syncthreads();
    }
    float* out = y + (size_t)blockIdx.z * plane;
    const int p0 = first + quad, p1 = p0 + 8;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int c = c0 + warp * 16 + 8 * j + pair;
        if (c < width) {                                // width is even
            if (p0 < last) *reinterpret_cast<float2*>(out + (size_t)p0 * width + c) = make_float2(acc[j][0], acc[j][1]);
            if (p1 < last) *reinterpret_cast<float2*>(out + (size_t)p1 * width + c) = make_float2(acc[j][2], acc[j][3]);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// And for prompts that bring an expert a hundred tokens and more: tiles of 128 places x 128 outputs (with a gate: 64
// outputs, their gate rows and their up rows side by side as the tile's 128 weight rows), eight warps in two rows of four,
// a warp 64 places x 32 weight rows in registers, the reduction in slices of 64 lanes through three buffers.  A warp
// issues 16 mma for 6 ldmatrix where the 64-place kernels issue 8 for 5, and a weight row fetched from L2 serves twice
// the places.
// ---------------------------------------------------------------------------------------------
constexpr int kWM = 128, kWN = 128, kWK = 64, kWStride = kWK + 8, kWStages = 3;
constexpr int kWTile = kWM * kWStride;
#ifndef BLM_MOE_WIDE_PAIRS
#define BLM_MOE_WIDE_PAIRS 96        // from this many (token, expert) pairs an expert on average the wide kernels run
#endif

// one slice: acc[mi][ni] += x (64 places of the warp) . w (the warp's 32 weight rows: two runs of 16 at rb0 and rb1)
__device__ __forceinline__ void moe_wide_slice(float (&acc)[4][4][4], unsigned xs, unsigned ws, int wm, int rb0, int rb1, int lrow, int lmat) {
#pragma unroll
    for (int kk = 0; kk < kWK; kk += 16) {
        uint32_t a[4][4], b0[4], b1[4];
#pragma unroll
        for (int mi = 0; mi < 4; ++mi)
            moe_ldsm_x4(a[mi], xs + ((wm * 64 + mi * 16 + lrow + (lmat & 1) * 8) * kWStride + kk + (lmat >> 1) * 8) * 2);
        moe_ldsm_x4(b0, ws + ((rb0 + lrow + (lmat >> 1) * 8) * kWStride + kk + (lmat & 1) * 8) * 2);
        moe_ldsm_x4(b1, ws + ((rb1 + lrow + (lmat >> 1) * 8) * kWStride + kk + (lmat & 1) * 8) * 2);
#pragma unroll
        for (int mi = 0; mi < 4; ++mi) {
            moe_mma(acc[mi][0], a[mi], b0[0], b0[1]);
            moe_mma(acc[mi][1], a[mi], b0[2], b0[3]);
            moe_mma(acc[mi][2], a[mi], b1[0], b1[1]);
            moe_mma(acc[mi][3], a[mi], b1[2], b1[3]);
        }
    }
}

template <bool kGated>
__global__ void __launch_bounds__(256) moe_up_wide_kernel(const __nv_bfloat16* __restrict__ h, const float* __restrict__ weights,
                                                          const int* __restrict__ order, const int* __restrict__ offsets,
                                                          const __nv_bfloat16* __restrict__ w_gu, __nv_bfloat16* __restrict__ act,
                                                          int width, int ff, int n_experts, int top, int scale_input, GluAct glu) {
    extern __shared__ __align__(16) unsigned char moe_smem[];
    __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(moe_smem);      // kWStages x (x [128], weight rows [128])
    __shared__ int token_of[kWM];
    __shared__ float scale_of[kWM];
    int e, first, last;
    if (!moe_find_tile(offsets, n_experts, blockIdx.x, &e, &first, &last, kWM)) return;
    constexpr int kOut = kGated ? kWN / 2 : kWN;           // outputs of a tile
    const int c0 = blockIdx.y * kOut;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, quad = lane >> 2, pair = (lane & 3) * 2;
    const int lrow = lane & 7, lmat = lane >> 3, wm = warp >> 2, wn = warp & 3;
    if (threadIdx.x < kWM) {
        const int place = first + threadIdx.x;
        int tok = -1;
        float sc = 1.f;
        if (place < last) {
            const int p = order[place];
            tok = p / top;
            if (scale_input) sc = weights[p];
        }
        token_of[threadIdx.x] = tok;
        scale_of[threadIdx.x] = sc;
    }
    __syncthreads();
    const __nv_bfloat16* wg = w_gu + (size_t)e * (kGated ? 2 : 1) * ff * width;
    auto stage_slice = [&](int buf, int k0) {
        __nv_bfloat16* xs = stage + buf * 2 * kWTile;
        for (int idx = threadIdx.x; idx < kWM * (kWK / 8); idx += blockDim.x) {
            const int r = idx / (kWK / 8), kk = (idx % (kWK / 8)) * 8;
            const int tok = token_of[r];
            const bool in = tok >= 0 && k0 + kk < width;
            moe_cp16(xs + r * kWStride + kk, in ? h + (size_t)tok * width + k0 + kk : h, in);
        }
        for (int idx = threadIdx.x; idx < kWN * (kWK / 8); idx += blockDim.x) {
            const int r = idx / (kWK / 8), kk = (idx % (kWK / 8)) * 8;
            // with a gate: rows 0 .. 63 the gate rows of the tile's outputs, rows 64 .. 127 their up rows (ff rows further on)
            const int c = kGated ? c0 + (r & (kOut - 1)) : c0 + r;
            const bool in = c < ff && k0 + kk < width;
            const size_t row = kGated && r >= kOut ? (size_t)ff + c : (size_t)c;
            moe_cp16(xs + kWTile + r * kWStride + kk, in ? wg + row * width + k0 + kk : wg, in);
        }
    };
    float acc[4][4][4];
#pragma unroll
    for (int mi = 0; mi < 4; ++mi)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) acc[mi][ni][0] = acc[mi][ni][1] = acc[mi][ni][2] = acc[mi][ni][3] = 0.f;
    const int rb0 = kGated ? wn * 16 : wn * 32, rb1 = kGated ? kOut + wn * 16 : wn * 32 + 16;
    const unsigned stage_at = (unsigned)__cvta_generic_to_shared(stage);
    const int n_slices = (width + kWK - 1) / kWK;
#pragma unroll
    for (int ahead = 0; ahead < kWStages - 1; ++ahead) {
        if (ahead < n_slices) stage_slice(ahead, ahead * kWK);
        moe_cp_commit();
    }
    for (int it = 0; it < n_slices; ++it) {
        const int buf = it % kWStages;
        if (it + kWStages - 1 < n_slices) stage_slice((it + kWStages - 1) % kWStages, (it + kWStages - 1) * kWK);
        moe_cp_commit();
        moe_cp_wait_all_but<kWStages - 1>();
        __syncthreads();
        const unsigned xs = stage_at + buf * 2 * kWTile * 2;
        moe_wide_slice(acc, xs, xs + kWTile * 2, wm, rb0, rb1, lrow, lmat);
        __syncthreads();
    }
#pragma unroll
    for (int mi = 0; mi < 4; ++mi)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = wm * 64 + mi * 16 + quad + 8 * half, place = first + r;
            if (place >= last) continue;
            const float sc = scale_of[r];
            if (kGated) {
#pragma unroll
                for (int ni = 0; ni < 2; ++ni) {
                    const int c = c0 + wn * 16 + 8 * ni + pair;
                    if (c < ff)
                        *reinterpret_cast<__nv_bfloat162*>(act + (size_t)place * ff + c) = __floats2bfloat162_rn(
                            glu_act(sc * acc[mi][ni][2 * half], sc * acc[mi][ni + 2][2 * half], glu),
                            glu_act(sc * acc[mi][ni][2 * half + 1], sc * acc[mi][ni + 2][2 * half + 1], glu));
                }
            } else {
#pragma unroll
                for (int ni = 0; ni < 4; ++ni) {
                    const int c = c0 + wn * 32 + 8 * ni + pair;
                    if (c < ff)
                        *reinterpret_cast<__nv_bfloat162*>(act + (size_t)place * ff + c) = __floats2bfloat162_rn(
                            glu_act(sc * acc[mi][ni][2 * half], 0.f, glu), glu_act(sc * acc[mi][ni][2 * half + 1], 0.f, glu));
                }
            }
        }
}

__global__ void __launch_bounds__(256) moe_down_wide_kernel(const __nv_bfloat16* __restrict__ act, const int* __restrict__ offsets,
                                                            const __nv_bfloat16* __restrict__ w_down, float* __restrict__ y, int width, int ff,
                                                            int n_experts) {
    extern __shared__ __align__(16) unsigned char moe_smem[];
    __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(moe_smem);      // kWStages x (x [128], weight rows [128])
    int e, first, last;
    if (!moe_find_tile(offsets, n_experts, blockIdx.x, &e, &first, &last, kWM)) return;
    const int c0 = blockIdx.y * kWN;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, quad = lane >> 2, pair = (lane & 3) * 2;
    const int lrow = lane & 7, lmat = lane >> 3, wm = warp >> 2, wn = warp & 3;
    const __nv_bfloat16* wd = w_down + (size_t)e * width * ff;
    auto stage_slice = [&](int buf, int k0) {
        __nv_bfloat16* xs = stage + buf * 2 * kWTile;
        for (int idx = threadIdx.x; idx < kWM * (kWK / 8); idx += blockDim.x) {
            const int r = idx / (kWK / 8), kk = (idx % (kWK / 8)) * 8;
            const bool in = first + r < last && k0 + kk < ff;
            moe_cp16(xs + r * kWStride + kk, in ? act + (size_t)(first + r) * ff + k0 + kk : act, in);
        }
        for (int idx = threadIdx.x; idx < kWN * (kWK / 8); idx += blockDim.x) {
            const int r = idx / (kWK / 8), kk = (idx % (kWK / 8)) * 8;
            const bool in = c0 + r < width && k0 + kk < ff;
            moe_cp16(xs + kWTile + r * kWStride + kk, in ? wd + (size_t)(c0 + r) * ff + k0 + kk : wd, in);
        }
    };
    float acc[4][4][4];
#pragma unroll
    for (int mi = 0; mi < 4; ++mi)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) acc[mi][ni][0] = acc[mi][ni][1] = acc[mi][ni][2] = acc[mi][ni][3] = 0.f;
    const unsigned stage_at = (unsigned)__cvta_generic_to_shared(stage);
    const int n_slices = (ff + kWK - 1) / kWK;
#pragma unroll
    for (int ahead = 0; ahead < kWStages - 1; ++ahead) {
        if (ahead < n_slices) stage_slice(ahead, ahead * kWK);
        moe_cp_commit();
    }
    for (int it = 0; it < n_slices; ++it) {
        const int buf = it % kWStages;
        if (it + kWStages - 1 < n_slices) stage_slice((it + kWStages - 1) % kWStages, (it + kWStages - 1) * kWK);
        moe_cp_commit();
        moe_cp_wait_all_but<kWStages - 1>();
        __syncthreads();
        const unsigned xs = stage_at + buf * 2 * kWTile * 2;
        moe_wide_slice(acc, xs, xs + kWTile * 2, wm, wn * 32, wn * 32 + 16, lrow, lmat);
        __syncthreads();
    }
#pragma unroll
    for (int mi = 0; mi < 4; ++mi)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int place = first + wm * 64 + mi * 16 + quad + 8 * half;
            if (place >= last) continue;
#pragma unroll
            for (int ni = 0; ni < 4; ++ni) {
                const int c = c0 + wn * 32 + 8 * ni + pair;
                if (c < width) *reinterpret_cast<float2*>(y + (size_t)place * width + c) = make_float2(acc[mi][ni][2 * half], acc[mi][ni][2 * half + 1]);
            }
        }
}

static bool moe_runs_wide(int dtype, long long pairs, int width, int ff, int n_experts) {
    return dtype == BLM_BF16 && width % 8 == 0 && ff % 8 == 0 && pairs >= (long long)BLM_MOE_WIDE_PAIRS * n_experts;
}

static bool moe_runs_skinny(int dtype, long long pairs, int width, int ff, int n_experts) {
    return dtype == BLM_BF16 && width % 8 == 0 && ff % 8 == 0 && pairs <= (long long)BLM_MOE_SKINNY_PAIRS * n_experts;
}

// Over how many blocks the second product's reduction is cut (the planes of y the caller provides): 1 unless the skinny
// kernels run and their tiles of places x output tiles would leave most multiprocessors without a block.
BLM_API int blm_moe_down_splits(int dtype, int n_tokens, int width, int ff, int n_experts, int top) {
    const long long pairs = (long long)n_tokens * top;
    if (!moe_runs_skinny(dtype, pairs, width, ff, n_experts)) return 1;
    const long long busy = (pairs < n_experts ? pairs : n_experts) + pairs / kSM;      // tiles of places that have a place
    const long long blocks = busy * ((width + kSN - 1) / kSN);
    long long splits = (4 * 148 + blocks - 1) / blocks;
    const long long most = (ff + 4 * kSK - 1) / (4 * kSK);                             // four slices a block at least
    if (splits > most) splits = most;
    if (splits > 16) splits = 16;
    return splits < 1 ? 1 : (int)splits;
}

BLM_API int blm_moe_experts(const void* h, int dtype, const float* weights, const int* order, const int* offsets, const void* w_gu,
                            const void* w_down, void* act, float* y, int n_tokens, int width, int ff, int n_experts, int top,
                            int scale_input, float act_limit, float act_alpha, int plain_unit, int down_splits, cudaStream_t stream) {
    // down_splits: blm_moe_down_splits(...) of the same sizes; y holds that many planes [places][width]
    // plain_unit 0: the gated units, w_gu [experts][2 ff][width]; act_limit <= 0: silu(gate) * up; > 0: the clamped unit with
    // that limit and act_alpha.  plain_unit 1 (exact GELU) or 2 (tanh GELU): no gate, w_gu [experts][ff][width]
    if (n_tokens == 0) return BLM_OK;
    BLM_REQUIRE(n_tokens > 0 && width > 0 && ff > 0 && n_experts > 0 && top > 0, "moe_experts: bad sizes");
    BLM_REQUIRE(plain_unit >= 0 && plain_unit <= 2, "moe_experts: unit %d", plain_unit);
    const GluAct glu{act_limit, act_alpha, plain_unit};
    const long long pairs = (long long)n_tokens * top;
    const long long tiles = (pairs + kBM - 1) / kBM + n_experts;      // every expert's share may end in a tile that is not full
    BLM_REQUIRE(tiles < (1ll << 31), "moe_experts: %lld tiles", tiles);
    const dim3 g1((unsigned)tiles, (unsigned)((ff + kBN - 1) / kBN)), g2((unsigned)tiles, (unsigned)((width + kBN - 1) / kBN));
    BLM_REQUIRE(g1.y <= 65535 && g2.y <= 65535, "moe_experts: too many output tiles");
    BLM_REQUIRE(down_splits == blm_moe_down_splits(dtype, n_tokens, width, ff, n_experts, top), "moe_experts: %d planes of sums", down_splits);
    if (moe_runs_skinny(dtype, pairs, width, ff, n_experts)) {
        const long long t16 = (pairs + kSM - 1) / kSM + n_experts;
        const dim3 s1((unsigned)t16, (unsigned)((ff + kSN - 1) / kSN)), s2((unsigned)t16, (unsigned)((width + kSN - 1) / kSN), (unsigned)down_splits);
        BLM_REQUIRE(s1.y <= 65535 && s2.y <= 65535, "moe_experts: too many output tiles");
        const int smem_up = 2 * (kSTileX + (plain_unit ? 1 : 2) * kSTileW) * (int)sizeof(__nv_bfloat16);
        const int smem_down = 2 * (kSTileX + kSTileW) * (int)sizeof(__nv_bfloat16);
        auto up_kernel = plain_unit ? moe_up_skinny_kernel<false> : moe_up_skinny_kernel<true>;
        cudaError_t err = cudaFuncSetAttribute(up_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_up);
        if (err != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "moe_experts: %s", cudaGetErrorString(err));
        up_kernel<<<s1, 128, smem_up, stream>>>((const __nv_bfloat16*)h, weights, order, offsets, (const __nv_bfloat16*)w_gu,
                                                (__nv_bfloat16*)act, width, ff, n_experts, top, scale_input, glu);
        moe_down_skinny_kernel<<<s2, 128, smem_down, stream>>>((const __nv_bfloat16*)act, offsets, (const __nv_bfloat16*)w_down, y, width, ff,
                                                               n_experts, pairs * width);
        return blm_check_launch("moe_experts (few tokens an expert)");
    }
    if (moe_runs_wide(dtype, pairs, width, ff, n_experts)) {
        const long long t128 = (pairs + kWM - 1) / kWM + n_experts;
        const int outs = plain_unit ? kWN : kWN / 2;
        const dim3 w1((unsigned)t128, (unsigned)((ff + outs - 1) / outs)), w2((unsigned)t128, (unsigned)((width + kWN - 1) / kWN));
        BLM_REQUIRE(w1.y <= 65535 && w2.y <= 65535, "moe_experts: too many output tiles");
        const int smem = kWStages * 2 * kWTile * (int)sizeof(__nv_bfloat16);
        auto up_kernel = plain_unit ? moe_up_wide_kernel<false> : moe_up_wide_kernel<true>;
        cudaError_t err = cudaFuncSetAttribute(up_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (err == cudaSuccess) err = cudaFuncSetAttribute(moe_down_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (err != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "moe_experts: %s", cudaGetErrorString(err));
        up_kernel<<<w1, 256, smem, stream>>>((const __nv_bfloat16*)h, weights, order, offsets, (const __nv_bfloat16*)w_gu,
                                             (__nv_bfloat16*)act, width, ff, n_experts, top, scale_input, glu);
        moe_down_wide_kernel<<<w2, 256, smem, stream>>>((const __nv_bfloat16*)act, offsets, (const __nv_bfloat16*)w_down, y, width, ff,
                                                        n_experts);
        return blm_check_launch("moe_experts (many tokens an expert)");
    }
    if (dtype == BLM_F32) {
        moe_gate_up_kernel<float><<<g1, 256, 0, stream>>>((const float*)h, weights, order, offsets, (const float*)w_gu, (float*)act, width,
                                                          ff, n_experts, top, scale_input, glu);
        moe_down_kernel<float><<<g2, 256, 0, stream>>>((const float*)act, offsets, (const float*)w_down, y, width, ff, n_experts);
    } else if (dtype == BLM_BF16 && width % 8 == 0 && ff % 8 == 0) {
        const long long t64 = (pairs + kTM - 1) / kTM + n_experts;
        const dim3 t1((unsigned)t64, (unsigned)((ff + kTN - 1) / kTN)), t2((unsigned)t64, (unsigned)((width + kTN - 1) / kTN));
        const int smem1 = kMoeStages * (plain_unit ? 2 : 3) * kTile * (int)sizeof(__nv_bfloat16);
        const int smem2 = kMoeStages * 2 * kTile * (int)sizeof(__nv_bfloat16);
        auto up_kernel = plain_unit ? moe_gate_up_tc_kernel<false> : moe_gate_up_tc_kernel<true>;
        cudaError_t err = cudaFuncSetAttribute(up_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1);
        if (err != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "moe_experts: %s", cudaGetErrorString(err));
        up_kernel<<<t1, 128, smem1, stream>>>((const __nv_bfloat16*)h, weights, order, offsets, (const __nv_bfloat16*)w_gu,
                                              (__nv_bfloat16*)act, width, ff, n_experts, top, scale_input, glu);
        err = cudaFuncSetAttribute(moe_down_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2);
        if (err != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "moe_experts: %s", cudaGetErrorString(err));
        moe_down_tc_kernel<<<t2, 128, smem2, stream>>>((const __nv_bfloat16*)act, offsets, (const __nv_bfloat16*)w_down, y, width, ff,
                                                       n_experts);
    } else if (dtype == BLM_BF16) {
        moe_gate_up_kernel<__nv_bfloat16><<<g1, 256, 0, stream>>>((const __nv_bfloat16*)h, weights, order, offsets,
                                                                  (const __nv_bfloat16*)w_gu, (__nv_bfloat16*)act, width, ff, n_experts,
                                                                  top, scale_input, glu);
        moe_down_kernel<__nv_bfloat16><<<g2, 256, 0, stream>>>((const __nv_bfloat16*)act, offsets, (const __nv_bfloat16*)w_down, y, width,
                                                               ff, n_experts);
    } else {
        return blm_fail(BLM_BAD_ARGUMENT, "moe_experts: dtype %d", dtype);
    }
    return blm_check_launch("moe_experts");
}

// ---------------------------------------------------------------------------------------------
// For the grouped product on tcgen05 (gemm_tc.cu): the pairs laid out expert by expert with every expert's share starting at
// a multiple of `tile_rows` places.  place_of[pair] = its place; pair_of_place[place] = the pair, -1 for a place no pair
// owns; tile_expert[tile] = the expert that owns the tile of places, -1 for none.  One block.
// ---------------------------------------------------------------------------------------------
__global__ void moe_group_padded_kernel(const int* __restrict__ ids, int n_pairs, int n_experts, int tile_rows, int max_tiles,
                                        int* __restrict__ place_of, int* __restrict__ pair_of_place, int* __restrict__ tile_expert) {
    extern __shared__ int counts[];      // [n_experts] counts, then [n_experts] cursors
    int* cursor = counts + n_experts;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
    for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) tile_expert[t] = -1;
    for (int p = threadIdx.x; p < max_tiles * tile_rows; p += blockDim.x) pair_of_place[p] = -1;
    __syncthreads();
    for (int a = threadIdx.x; a < n_pairs; a += blockDim.x) atomicAdd(&counts[min(max(ids[a], 0), n_experts - 1)], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int tile = 0;
        for (int e = 0; e < n_experts; ++e) {
            cursor[e] = tile * tile_rows;
            const int tiles = (counts[e] + tile_rows - 1) / tile_rows;
            for (int t = 0; t < tiles && tile + t < max_tiles; ++t) tile_expert[tile + t] = e;
            tile += tiles;
        }
    }
    __syncthreads();
    for (int a = threadIdx.x; a < n_pairs; a += blockDim.x) {
        const int place = atomicAdd(&cursor[min(max(ids[a], 0), n_experts - 1)], 1);
        place_of[a] = place;
        pair_of_place[place] = a;
    }
}

// xs[place] = h[token of the place's pair] (zeros for a place no pair owns), 16 bytes a thread and step
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ h, const int* __restrict__ pair_of_place, __nv_bfloat16* __restrict__ xs,
                                       int width, int top) {
    const int place = blockIdx.x;
    const int pair = pair_of_place[place];
    const uint4* src = pair >= 0 ? reinterpret_cast<const uint4*>(h + (size_t)(pair / top) * width) : nullptr;
    uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)place * width);
    for (int i = threadIdx.x; i < width / 8; i += blockDim.x) dst[i] = src ? src[i] : make_uint4(0, 0, 0, 0);
}

// How many tiles of `tile_rows` places the padded layout of n_pairs pairs over n_experts experts can take at most.
BLM_API int blm_moe_padded_tiles(int n_pairs, int n_experts, int tile_rows) { return (n_pairs + tile_rows - 1) / tile_rows + n_experts; }

BLM_API int blm_moe_group_padded(const int* ids, int n_pairs, int n_experts, int tile_rows, int* place_of, int* pair_of_place,
                                 int* tile_expert, cudaStream_t stream) {
    if (n_pairs == 0) return BLM_OK;
    BLM_REQUIRE(n_pairs > 0 && n_experts > 0 && n_experts <= 4096 && tile_rows > 0, "moe_group_padded: bad sizes");
    const int max_tiles = blm_moe_padded_tiles(n_pairs, n_experts, tile_rows);
    moe_group_padded_kernel<<<1, 1024, 2 * (size_t)n_experts * sizeof(int), stream>>>(ids, n_pairs, n_experts, tile_rows, max_tiles, place_of,
                                                                                      pair_of_place, tile_expert);
    return blm_check_launch("moe_group_padded");
}

BLM_API int blm_moe_gather_rows(const void* h, const int* pair_of_place, void* xs, int n_places, int width, int top, cudaStream_t stream) {
    if (n_places == 0) return BLM_OK;
    BLM_REQUIRE(n_places > 0 && width > 0 && width % 8 == 0 && top > 0, "moe_gather_rows: bad sizes");
    BLM_REQUIRE((((size_t)h | (size_t)xs) & 15) == 0, "moe_gather_rows: rows must be 16-byte aligned");
    moe_gather_rows_kernel<<<n_places, 128, 0, stream>>>((const __nv_bfloat16*)h, pair_of_place, (__nv_bfloat16*)xs, width, top);
    return blm_check_launch("moe_gather_rows");
}

// ---------------------------------------------------------------------------------------------
// out[n] = sum_k (weight_k if the weight is on the output) y[place_of[n, k]] + extra[n]   (k in the order of the choice);
// y may come in n_planes planes of [places][width] whose sum it is
// ---------------------------------------------------------------------------------------------
template <typename T, typename TO>
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ place_of, const float* __restrict__ weights,
                                   const T* __restrict__ extra, TO* __restrict__ out, int width, int top, int scale_output, int n_planes,
                                   long long plane) {
    const int n = blockIdx.x;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k) {
            const size_t at = (size_t)place_of[(size_t)n * top + k] * width + d;
            float v = y[at];
            for (int z = 1; z < n_planes; ++z) v += y[at + (size_t)z * plane];      // the shares of a cut reduction, in order
            s += scale_output ? weights[(size_t)n * top + k] * v : v;
        }
        if (extra) s += to_f32(extra[(size_t)n * width + d]);
        out[(size_t)n * width + d] = from_f32<TO>(s);
    }
}

BLM_API int blm_moe_combine(const float* y, const int* place_of, const float* weights, const void* extra, void* out, int dtype,
                            int n_tokens, int width, int top, int scale_output, int out_dtype, int n_planes, cudaStream_t stream) {
    // dtype: that of `extra`; out_dtype: that of `out` (the same, or float32: the sum handed on unrounded)
    if (n_tokens == 0) return BLM_OK;
    BLM_REQUIRE(n_tokens > 0 && width > 0 && top > 0 && n_planes >= 1, "moe_combine: bad sizes");
    const long long plane = (long long)n_tokens * top * width;
    if (dtype == BLM_BF16 && out_dtype == BLM_F32)
        moe_combine_kernel<__nv_bfloat16, float><<<n_tokens, 256, 0, stream>>>(y, place_of, weights, (const __nv_bfloat16*)extra,
                                                                               (float*)out, width, top, scale_output, n_planes, plane);
    else if (dtype != out_dtype)
        return blm_fail(BLM_BAD_ARGUMENT, "moe_combine: dtype %d with out dtype %d", dtype, out_dtype);
    else if (dtype == BLM_F32)
        moe_combine_kernel<float, float><<<n_tokens, 256, 0, stream>>>(y, place_of, weights, (const float*)extra, (float*)out, width, top, scale_output, n_planes, plane);
    else if (dtype == BLM_BF16)
        moe_combine_kernel<__nv_bfloat16, __nv_bfloat16><<<n_tokens, 256, 0, stream>>>(y, place_of, weights, (const __nv_bfloat16*)extra,
                                                                                       (__nv_bfloat16*)out, width, top, scale_output, n_planes, plane);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "moe_combine: dtype %d", dtype);
    return blm_check_launch("moe_combine");
}
