// Sparse mixture-of-experts feed-forward without host synchronisation: router, expert GEMVs that follow the expert
// index on the device ("selective loading": only the chosen experts' weights are touched), clamped gated activation,
// and the weighted combination in fp32.  bf16 or fp32 activations / expert weights; router in fp32.
//
//   router        z = Wr h (+ logit bias);  s = softmax(z);  choice = s + correction;  the `top` largest choices are taken,
//                 weight = s * out_scale (not renormalised);  optional second output sigmoid(<w_sg, h>) per token.
//                 renormalise: the `top` largest LOGITS are taken and the weights are the softmax over the chosen
//                 logits only (times out_scale)
//                 sigmoid scores (mode 2): s = sigmoid(z) per expert instead of the softmax, otherwise as the first form
//   activation    g = min(gate, limit), u = clamp(up, -limit, limit);  a = g * sigmoid(alpha * g) * (u + up_shift)
//                 (limit = +inf, alpha = 1, up_shift = 0: plain silu(gate) * up)
//   expert index >= E means an identity expert: its output is the token's input itself
// Expert weights are stored [E, in, out] (the layout of the grouped expert layers), gate | up fused on the out dim.
#include "common.cuh"

namespace {

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ void ld2(const float* p, float& a, float& b) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    a = v.x;
    b = v.y;
}
__device__ __forceinline__ void ld2(const bf16* p, float& a, float& b) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const bf162*>(p));
    a = v.x;
    b = v.y;
}

// kind 0: g * sigmoid(alpha g); kind 1: the tanh form of gelu, 0.5 g (1 + tanh(c (g + 0.044715 g^3))) with c = sqrt(2 / pi),
// written through 0.5 (1 + tanh(a)) = sigmoid(2 a)
__device__ __forceinline__ float glu_act(float g, float u, float limit, float alpha, float up_shift, int kind = 0) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    const float a = kind == 1 ? 1.5957691216057308f * (g + 0.044715f * g * g * g) : alpha * g;
    return g / (1.f + expf(-a)) * (u + up_shift);
}

// ---- router ---------------------------------------------------------------------------------------------------------
constexpr int RT_WARPS = 4, RT_GROUP = 8;

template <typename T>
__global__ void __launch_bounds__(RT_WARPS * 32)
moe_router_kernel(const T* __restrict__ h, const float* __restrict__ wr, const float* __restrict__ corr,
                  const float* __restrict__ wsg, int* __restrict__ idx, float* __restrict__ wts,
                  float* __restrict__ sgate, long long N, int W, int R, int top, float out_scale,
                  const float* __restrict__ zbias, int mode) {
    extern __shared__ float smem[];
    const bool renorm = mode == 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* ps = smem + (long long)warp * 2 * R;     // probabilities
    float* cs = ps + R;                             // choice scores
    const long long n = (long long)blockIdx.x * RT_WARPS + warp;
    if (n >= N) return;
    const T* hr = h + n * W;
    for (int r0 = 0; r0 < R; r0 += RT_GROUP) {
        float acc[RT_GROUP];
#pragma unroll
        for (int i = 0; i < RT_GROUP; ++i) acc[i] = 0.f;
        for (int c = lane; c < W; c += 32) {
            const float hv = ldf(hr + c);
#pragma unroll
            for (int i = 0; i < RT_GROUP; ++i)
                if (r0 + i < R) acc[i] = fmaf(hv, wr[(long long)(r0 + i) * W + c], acc[i]);
        }
#pragma unroll
        for (int i = 0; i < RT_GROUP; ++i) {
            const float z = warp_sum(acc[i]);
            if (lane == 0 && r0 + i < R) ps[r0 + i] = z + (zbias != nullptr ? zbias[r0 + i] : 0.f);
        }
    }
    if (wsg != nullptr && sgate != nullptr) {
        float a = 0.f;
        for (int c = lane; c < W; c += 32) a = fmaf(ldf(hr + c), wsg[c], a);
        a = warp_sum(a);
        if (lane == 0) sgate[n] = 1.f / (1.f + expf(-a));
    }
    __syncwarp();
    if (renorm) {                // the choice is made on the logits themselves
        for (int r = lane; r < R; r += 32) cs[r] = ps[r];
    } else if (mode == 2) {      // independent sigmoid scores
        for (int r = lane; r < R; r += 32) {
            const float p = 1.f / (1.f + expf(-ps[r]));
            ps[r] = p;
            cs[r] = p + (corr != nullptr ? corr[r] : 0.f);
        }
    } else {
        float mx = -INFINITY;
        for (int r = lane; r < R; r += 32) mx = fmaxf(mx, ps[r]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int r = lane; r < R; r += 32) sum += expf(ps[r] - mx);
        sum = warp_sum(sum);
        const float inv = 1.f / sum;
        __syncwarp();
        for (int r = lane; r < R; r += 32) {
            const float p = expf(ps[r] - mx) * inv;
            ps[r] = p;
            cs[r] = p + (corr != nullptr ? corr[r] : 0.f);
        }
    }
    __syncwarp();
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int r = lane; r < R; r += 32) {
            const float c = cs[r];
            if (c > best) {       // lanes scan upwards: the lowest index wins a tie inside a lane
                best = c;
                bi = r;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) {
                best = ob;
                bi = oi;
            }
        }
        if (bi >= R) bi = 0;      // every score NaN: keep the index in range
        if (lane == 0) {
            idx[n * top + k] = bi;
            wts[n * top + k] = renorm ? ps[bi] : ps[bi] * out_scale;
            cs[bi] = -INFINITY;
        }
        __syncwarp();
    }
    if (renorm && lane == 0) {   // softmax over the chosen logits only; the first pick is the largest
        const float mx = wts[n * top];
        float sum = 0.f;
        for (int k = 0; k < top; ++k) {
            const float e = expf(wts[n * top + k] - mx);
            wts[n * top + k] = e;
            sum += e;
        }
        const float inv = out_scale / sum;
        for (int k = 0; k < top; ++k) wts[n * top + k] *= inv;
    }
}

// ---- gate/up GEMV + activation for (token, expert) pairs ----------------------------------------------------------------
constexpr int GV_WARPS = 8;

template <typename T, bool VEC>
__global__ void __launch_bounds__(GV_WARPS * 32)
moe_gate_up_act_kernel(const T* __restrict__ h, const T* __restrict__ wgu, const int* __restrict__ idx,
                       T* __restrict__ act, int pairs_per_token, int W, int F, int E, float limit, float alpha,
                       float up_shift, const float* __restrict__ in_scale) {
    extern __shared__ float smem[];
    constexpr int PER = VEC ? 2 : 1, COLS = 32 * PER;
    float* hs = smem;                                  // [W]
    float* red = smem + W;                             // [GV_WARPS][COLS][2]
    const long long p = blockIdx.x;
    const int e = idx != nullptr ? idx[p] : 0;
    if (e < 0 || e >= E) return;                       // identity expert: no intermediate
    const long long t = p / pairs_per_token;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float xs = in_scale != nullptr ? in_scale[p] : 1.f;       // the pair's weight applied to the expert's INPUT
    for (int c = threadIdx.x; c < W; c += GV_WARPS * 32) hs[c] = ldf(h + t * W + c) * xs;
    __syncthreads();
    const int f0 = blockIdx.y * COLS + lane * PER;
    const int per = (W + GV_WARPS - 1) / GV_WARPS;
    const int k_lo = warp * per, k_hi = min(W, k_lo + per);
    float g0 = 0.f, g1 = 0.f, u0 = 0.f, u1 = 0.f;
    if (f0 < F) {
        const T* base = wgu + (long long)e * W * 2 * F;
#pragma unroll 4
        for (int k = k_lo; k < k_hi; ++k) {
            const T* row = base + (long long)k * 2 * F;
            const float hv = hs[k];
            if (VEC) {
                float a, b, c, d;
                ld2(row + f0, a, b);
                ld2(row + F + f0, c, d);
                g0 = fmaf(hv, a, g0);
                g1 = fmaf(hv, b, g1);
                u0 = fmaf(hv, c, u0);
                u1 = fmaf(hv, d, u1);
            } else {
                g0 = fmaf(hv, ldf(row + f0), g0);
                u0 = fmaf(hv, ldf(row + F + f0), u0);
            }
        }
    }
    float* mine = red + ((long long)warp * COLS + lane * PER) * 2;
    mine[0] = g0;
    mine[1] = u0;
    if (VEC) {
        mine[2] = g1;
        mine[3] = u1;
    }
    __syncthreads();
    if (threadIdx.x < COLS) {
        const int f = blockIdx.y * COLS + threadIdx.x;
        if (f < F) {
            float g = 0.f, u = 0.f;
#pragma unroll
            for (int w = 0; w < GV_WARPS; ++w) {
                g += red[((long long)w * COLS + threadIdx.x) * 2];
                u += red[((long long)w * COLS + threadIdx.x) * 2 + 1];
            }
            stf(act + p * F + f, glu_act(g, u, limit, alpha, up_shift));
        }
    }
}

// ---- down GEMV + weighted combination (+ identity experts, + gated shared expert) -> fp32 ---------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(GV_WARPS * 32)
moe_down_combine_kernel(const T* __restrict__ act, const T* __restrict__ wd, const int* __restrict__ idx,
                        const float* __restrict__ wts, const T* __restrict__ h, const T* __restrict__ act_s,
                        const T* __restrict__ wds, const float* __restrict__ sgate, float* __restrict__ y, int top, int W,
                        int F, int Fs, int E) {
    constexpr int PER = VEC ? 2 : 1, COLS = 32 * PER;
    __shared__ float red[GV_WARPS][COLS];
    const long long t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c0 = blockIdx.y * COLS + lane * PER;
    float a0 = 0.f, a1 = 0.f;
    if (c0 < W) {
        for (int j = 0; j < top; ++j) {
            const int e = idx[t * top + j];
            const float wgt = wts[t * top + j];
            if (e < 0 || e >= E) {
                if (warp == 0) {
                    a0 = fmaf(wgt, ldf(h + t * W + c0), a0);
                    if (VEC) a1 = fmaf(wgt, ldf(h + t * W + c0 + 1), a1);
                }
                continue;
            }
            const T* arow = act + (t * top + j) * F;
            const T* base = wd + (long long)e * F * W;
            const int per = (F + GV_WARPS - 1) / GV_WARPS;
            const int f_lo = warp * per, f_hi = min(F, f_lo + per);
            float s0 = 0.f, s1 = 0.f;
#pragma unroll 4
            for (int f = f_lo; f < f_hi; ++f) {
                const float av = ldf(arow + f);
                if (VEC) {
                    float p, q;
                    ld2(base + (long long)f * W + c0, p, q);
                    s0 = fmaf(av, p, s0);
                    s1 = fmaf(av, q, s1);
                } else {
                    s0 = fmaf(av, ldf(base + (long long)f * W + c0), s0);
                }
            }
            a0 = fmaf(wgt, s0, a0);
            a1 = fmaf(wgt, s1, a1);
        }
        if (act_s != nullptr) {
            const float wgt = sgate != nullptr ? sgate[t] : 1.f;
            const T* arow = act_s + t * Fs;
            const int per = (Fs + GV_WARPS - 1) / GV_WARPS;
            const int f_lo = warp * per, f_hi = min(Fs, f_lo + per);
            float s0 = 0.f, s1 = 0.f;
#pragma unroll 4
            for (int f = f_lo; f < f_hi; ++f) {
                const float av = ldf(arow + f);
                if (VEC) {
                    float p, q;
                    ld2(wds + (long long)f * W + c0, p, q);
                    s0 = fmaf(av, p, s0);
                    s1 = fmaf(av, q, s1);
                } else {
                    s0 = fmaf(av, ldf(wds + (long long)f * W + c0), s0);
                }
            }
            a0 = fmaf(wgt, s0, a0);
            a1 = fmaf(wgt, s1, a1);
        }
    }
    red[warp][lane * PER] = a0;
    if (VEC) red[warp][lane * PER + 1] = a1;
    __syncthreads();
    if (threadIdx.x < COLS) {
        const int c = blockIdx.y * COLS + threadIdx.x;
        if (c < W) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < GV_WARPS; ++w) s += red[w][threadIdx.x];
            y[t * W + c] = s;
        }
    }
}

// ---- pieces of the sorted (GEMM) path: activation over [M, 2F], gather-combine -------------------------------------------
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ out, long long M, int F, float limit,
                                   float alpha, float up_shift) {
    const long long total = M * F;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long m = i / F;
        const int f = (int)(i - m * F);
        stf(out + i, glu_act(ldf(gu + m * 2 * F + f), ldf(gu + m * 2 * F + F + f), limit, alpha, up_shift));
    }
}

// gate and up are column ranges of a wider row (a fused projection output), each with an optional fp32 bias
template <typename T>
__global__ void glu_bias_kernel(const T* __restrict__ src, long long ld, int gate_off, int up_off,
                                const float* __restrict__ gb, const float* __restrict__ ub, T* __restrict__ out, long long M,
                                int F, float limit, float alpha, float up_shift, int kind) {
    const long long total = M * F;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long m = i / F;
        const int f = (int)(i - m * F);
        const float g = ldf(src + m * ld + gate_off + f) + (gb != nullptr ? gb[f] : 0.f);
        const float u = ldf(src + m * ld + up_off + f) + (ub != nullptr ? ub[f] : 0.f);
        stf(out + i, glu_act(g, u, limit, alpha, up_shift, kind));
    }
}

// the same with eight consecutive bf16 columns per thread (16-byte accesses, biases as two float4 each)
__global__ void glu_bias_vec_kernel(const bf16* __restrict__ src, long long ld, int gate_off, int up_off,
                                    const float* __restrict__ gb, const float* __restrict__ ub, bf16* __restrict__ out,
                                    long long M, int F8, float limit, float alpha, float up_shift, int kind) {
    const int f = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (f >= F8 * 8) return;
    float bg[8], bu[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) bg[j] = bu[j] = 0.f;
    if (gb != nullptr) {
        *reinterpret_cast<float4*>(bg) = *reinterpret_cast<const float4*>(gb + f);
        *reinterpret_cast<float4*>(bg + 4) = *reinterpret_cast<const float4*>(gb + f + 4);
    }
    if (ub != nullptr) {
        *reinterpret_cast<float4*>(bu) = *reinterpret_cast<const float4*>(ub + f);
        *reinterpret_cast<float4*>(bu + 4) = *reinterpret_cast<const float4*>(ub + f + 4);
    }
    for (long long m = blockIdx.y; m < M; m += gridDim.y) {
        float g[8], u[8], o[8];
        unpack8(*reinterpret_cast<const bf16x8*>(src + m * ld + gate_off + f), g);
        unpack8(*reinterpret_cast<const bf16x8*>(src + m * ld + up_off + f), u);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = glu_act(g[j] + bg[j], u[j] + bu[j], limit, alpha, up_shift, kind);
        *reinterpret_cast<bf16x8*>(out + m * F8 * 8 + f) = pack8(o);
    }
}

template <typename T>
__global__ void moe_gather_combine_kernel(const T* __restrict__ ys, const int* __restrict__ slot,
                                          const int* __restrict__ idx, const float* __restrict__ wts,
                                          const T* __restrict__ h, const T* __restrict__ shared_out,
                                          const float* __restrict__ sgate, float* __restrict__ y, int top, int W, int E) {
    const long long t = blockIdx.x;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float a = 0.f;
        for (int j = 0; j < top; ++j) {
            const int e = idx[t * top + j];
            const float wgt = wts[t * top + j];
            const float v = (e < 0 || e >= E) ? ldf(h + t * W + c) : ldf(ys + (long long)slot[t * top + j] * W + c);
            a = fmaf(wgt, v, a);
        }
        if (shared_out != nullptr) a = fmaf(sgate != nullptr ? sgate[t] : 1.f, ldf(shared_out + t * W + c), a);
        y[t * W + c] = a;
    }
}

}  // namespace

// dtype: 0 bf16, 1 fp32 (activations and expert weights).  R = router outputs (experts + identity experts).
// zbias [R] fp32 or NULL: added to the logits; mode 0: softmax scores; 1: choice on the logits, weights = softmax over the
// chosen ones; 2: sigmoid scores.
NXD_API int nxd_moe_router(int dtype, const void* h, const float* wr, const float* corr, const float* wsg, int* idx,
                           float* wts, float* sgate, long long N, int W, int R, int top, float out_scale,
                           const float* zbias, int mode, void* stream) {
    if (N == 0) return 0;
    NXD_REQUIRE(top >= 1 && top <= R, "router: top %d of %d", top, R);
    const size_t smem = (size_t)RT_WARPS * 2 * R * sizeof(float);
    NXD_REQUIRE(smem <= 48 * 1024, "router: %d outputs", R);
    const unsigned blocks = (unsigned)((N + RT_WARPS - 1) / RT_WARPS);
    if (dtype == 0)
        moe_router_kernel<bf16><<<blocks, RT_WARPS * 32, smem, (cudaStream_t)stream>>>((const bf16*)h, wr, corr, wsg, idx,
                                                                                      wts, sgate, N, W, R, top, out_scale,
                                                                                      zbias, mode);
    else
        moe_router_kernel<float><<<blocks, RT_WARPS * 32, smem, (cudaStream_t)stream>>>((const float*)h, wr, corr, wsg,
                                                                                       idx, wts, sgate, N, W, R, top,
                                                                                       out_scale, zbias, mode);
    NXD_LAUNCH_CHECK();
    return 0;
}

// act[p, :] = activation(h[p / pairs_per_token] @ wgu[idx[p]]) for P pairs; idx NULL = expert 0 for every pair (a dense
// gated MLP); pairs whose index is outside [0, E) are identity experts and are skipped.  in_scale [P] fp32 or NULL: the
// pair's input row is multiplied by it (routing weight on the expert's input).
NXD_API int nxd_moe_gate_up_act(int dtype, const void* h, const void* wgu, const int* idx, void* act, long long P,
                                int pairs_per_token, int W, int F, int E, float limit, float alpha, float up_shift,
                                const float* in_scale, void* stream) {
    if (P == 0) return 0;
    NXD_REQUIRE(P < (1ll << 31), "gate/up: %lld pairs", P);
    const bool vec = (F % 2) == 0;
    const int cols = vec ? 64 : 32;
    const size_t smem = (size_t)(W + GV_WARPS * cols * 2) * sizeof(float);
    NXD_REQUIRE(smem <= 200 * 1024, "gate/up: input width %d", W);
    dim3 grid((unsigned)P, (F + cols - 1) / cols);
    cudaStream_t st = (cudaStream_t)stream;
#define NXD_GU(T, V)                                                                                                  \
    do {                                                                                                              \
        auto kern = moe_gate_up_act_kernel<T, V>;                                                                     \
        if (smem > 48 * 1024)                                                                                         \
            NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));       \
        kern<<<grid, GV_WARPS * 32, smem, st>>>((const T*)h, (const T*)wgu, idx, (T*)act, pairs_per_token, W, F, E,   \
                                                limit, alpha, up_shift, in_scale);                                    \
    } while (0)
    if (dtype == 0) {
        if (vec) NXD_GU(bf16, true); else NXD_GU(bf16, false);
    } else {
        if (vec) NXD_GU(float, true); else NXD_GU(float, false);
    }
#undef NXD_GU
    NXD_LAUNCH_CHECK();
    return 0;
}

// y[t] = sum_j wts[t, j] * (idx[t, j] in [0, E) ? act[t * top + j] @ wd[idx[t, j]] : h[t])
//        + (act_s ? (sgate ? sgate[t] : 1) * act_s[t] @ wds : 0)                                  -> fp32 [N, W]
NXD_API int nxd_moe_down_combine(int dtype, const void* act, const void* wd, const int* idx, const float* wts,
                                 const void* h, const void* act_s, const void* wds, const float* sgate, float* y,
                                 long long N, int top, int W, int F, int Fs, int E, void* stream) {
    if (N == 0) return 0;
    NXD_REQUIRE(N < (1ll << 31), "down/combine: %lld tokens", N);
    const bool vec = (W % 2) == 0;
    const int cols = vec ? 64 : 32;
    dim3 grid((unsigned)N, (W + cols - 1) / cols);
    cudaStream_t st = (cudaStream_t)stream;
#define NXD_DC(T, V)                                                                                                  \
    moe_down_combine_kernel<T, V><<<grid, GV_WARPS * 32, 0, st>>>((const T*)act, (const T*)wd, idx, wts, (const T*)h, \
                                                                  (const T*)act_s, (const T*)wds, sgate, y, top, W, F,  \
                                                                  Fs, E)
    if (dtype == 0) {
        if (vec) NXD_DC(bf16, true); else NXD_DC(bf16, false);
    } else {
        if (vec) NXD_DC(float, true); else NXD_DC(float, false);
    }
#undef NXD_DC
    NXD_LAUNCH_CHECK();
    return 0;
}

NXD_API int nxd_clamped_glu(int dtype, const void* gate_up, void* out, long long M, int F, float limit, float alpha,
                            float up_shift, void* stream) {
    if (M == 0) return 0;
    long long blocks = (M * F + 255) / 256;
    const long long cap = (long long)nxd_num_sms() * 16;
    if (blocks > cap) blocks = cap;
    if (dtype == 0)
        clamped_glu_kernel<bf16><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const bf16*)gate_up, (bf16*)out, M, F,
                                                                                    limit, alpha, up_shift);
    else
        clamped_glu_kernel<float><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const float*)gate_up, (float*)out, M,
                                                                                     F, limit, alpha, up_shift);
    NXD_LAUNCH_CHECK();
    return 0;
}

// ys [pairs, W]: expert outputs in sorted order, slot [N, top]: row of ys of every (token, choice); identity experts read h.
NXD_API int nxd_moe_gather_combine(int dtype, const void* ys, const int* slot, const int* idx, const float* wts,
                                   const void* h, const void* shared_out, const float* sgate, float* y, long long N,
                                   int top, int W, int E, void* stream) {
    if (N == 0) return 0;
    NXD_REQUIRE(N < (1ll << 31), "combine: %lld tokens", N);
    if (dtype == 0)
        moe_gather_combine_kernel<bf16><<<(unsigned)N, 128, 0, (cudaStream_t)stream>>>(
            (const bf16*)ys, slot, idx, wts, (const bf16*)h, (const bf16*)shared_out, sgate, y, top, W, E);
    else
        moe_gather_combine_kernel<float><<<(unsigned)N, 128, 0, (cudaStream_t)stream>>>(
            (const float*)ys, slot, idx, wts, (const float*)h, (const float*)shared_out, sgate, y, top, W, E);
    NXD_LAUNCH_CHECK();
    return 0;
}

NXD_API int nxd_glu_bias(int dtype, const void* src, long long ld, int gate_off, int up_off, const float* gate_bias,
                         const float* up_bias, void* out, long long M, int F, float limit, float alpha, float up_shift,
                         int act_kind, void* stream) {
    if (M * F == 0) return 0;
    long long blocks = (M * F + 255) / 256;
    const long long cap = (long long)nxd_num_sms() * 16;
    if (blocks > cap) blocks = cap;
    if (dtype == 0 && F % 8 == 0 && ld % 8 == 0 && gate_off % 8 == 0 && up_off % 8 == 0 && ((uintptr_t)src % 16) == 0 &&
        ((uintptr_t)out % 16) == 0 && ((uintptr_t)gate_bias % 16) == 0 && ((uintptr_t)up_bias % 16) == 0) {
        const int F8 = F / 8, threads = F8 >= 256 ? 256 : ((F8 + 31) / 32) * 32;
        const long long rows_cap = (long long)nxd_num_sms() * 32;         // rows beyond that are walked by the same CTAs
        dim3 grid((F8 + threads - 1) / threads, (unsigned)(M < rows_cap ? M : rows_cap));
        glu_bias_vec_kernel<<<grid, threads, 0, (cudaStream_t)stream>>>((const bf16*)src, ld, gate_off, up_off, gate_bias,
                                                                        up_bias, (bf16*)out, M, F8, limit, alpha, up_shift,
                                                                        act_kind);
        NXD_LAUNCH_CHECK();
        return 0;
    }
    if (dtype == 0)
        glu_bias_kernel<bf16><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const bf16*)src, ld, gate_off, up_off,
                                                                                 gate_bias, up_bias, (bf16*)out, M, F, limit,
                                                                                 alpha, up_shift, act_kind);
    else
        glu_bias_kernel<float><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const float*)src, ld, gate_off, up_off,
                                                                                  gate_bias, up_bias, (float*)out, M, F,
                                                                                  limit, alpha, up_shift, act_kind);
    NXD_LAUNCH_CHECK();
    return 0;
}
