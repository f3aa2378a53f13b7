// Hyper-connections: the residual stream is S parallel streams x_1 .. x_S per token (fp32, [N, S, W]).  A sublayer reads a
// weighted sum of the streams and its output is written back into every stream, next to a learned mixing of the streams
// among themselves:
//
//   read    u = sum_s in[s] x_s;   h = u / sqrt(mean(u^2) + eps) * w            (RMS norm, h in the activation dtype)
//   write   x_t <- sum_s mix[s][t] x_s + out[t] * y      for all t at once, from the old streams
//
// y is the sublayer's output [N, W], or the mean of two branch outputs that are each RMS-normed over the width with a
// weight of their own:  y = 0.5 * (a / rms(a) * wa + b / rms(b) * wb).  S = 1 with in = mix = out = 1 is the plain
// pre-norm residual.
//
// One kernel does the write of one sublayer and the read of the next (either half may be absent): a CTA per token, the
// streams are read once and written once (four columns per thread through 16-byte accesses where widths and pointers
// allow), the weighted sum stays in shared memory between the two passes of the norm.
// Everything is fp32; this file is compiled without fast-math.
#include "common.cuh"

namespace {

constexpr int HC_MAX = 8, HC_THREADS = 256;

// loads / stores of VEC consecutive columns (VEC = 4: 16-byte fp32 and 8-byte bf16 accesses)
template <int VEC>
__device__ __forceinline__ void ldv(const float* p, float* v) {
    if (VEC == 4) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
    } else {
        v[0] = *p;
    }
}
template <int VEC>
__device__ __forceinline__ void ldv(const bf16* p, float* v) {
    if (VEC == 4) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const bf162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const bf162*>(&raw.y));
        v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
    } else {
        v[0] = __bfloat162float(*p);
    }
}
template <int VEC>
__device__ __forceinline__ void stv(float* p, const float* v) {
    if (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    else *p = v[0];
}
template <int VEC>
__device__ __forceinline__ void stv(bf16* p, const float* v) {
    if (VEC == 4) {
        uint2 raw;
        *reinterpret_cast<bf162*>(&raw.x) = __floats2bfloat162_rn(v[0], v[1]);
        *reinterpret_cast<bf162*>(&raw.y) = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(p) = raw;
    } else {
        *p = __float2bfloat16_rn(v[0]);
    }
}

// SMAX: most streams the instantiation holds in registers (S <= SMAX); VEC columns per thread and iteration.
template <typename TY, typename TH, int SMAX, int VEC>
__global__ void __launch_bounds__(HC_THREADS)
hc_step_kernel(float* __restrict__ X, const TY* __restrict__ ya, const TY* __restrict__ yb, const float* __restrict__ wa,
               const float* __restrict__ wb, const float* __restrict__ mix, const float* __restrict__ outw,
               const float* __restrict__ inw, const float* __restrict__ wn, TH* __restrict__ h, int S, int W, float eps) {
    extern __shared__ __align__(16) float us[];    // [W] the weighted sum of the (new) streams
    __shared__ float red[32];
    __shared__ float cm[HC_MAX * HC_MAX], co[HC_MAX], ci[HC_MAX];
    const long long n = blockIdx.x;
    const int tid = threadIdx.x;
    if (tid < S * S && mix != nullptr) cm[tid] = mix[tid];
    if (tid < S) {
        co[tid] = outw != nullptr ? outw[tid] : 0.f;
        ci[tid] = inw != nullptr ? inw[tid] : 0.f;
    }
    float* xr = X + n * S * W;
    const TY* ar = ya != nullptr ? ya + n * W : nullptr;
    const TY* br = yb != nullptr ? yb + n * W : nullptr;
    float ra = 1.f, rb = 1.f;
    if (br != nullptr) {                           // two normed branches: their root mean squares first
        float sa = 0.f, sb = 0.f;
        for (int c = tid * VEC; c < W; c += HC_THREADS * VEC) {
            float a[VEC], b[VEC];
            ldv<VEC>(ar + c, a);
            ldv<VEC>(br + c, b);
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                sa = fmaf(a[i], a[i], sa);
                sb = fmaf(b[i], b[i], sb);
            }
        }
        sa = block_sum(sa, red);
        sb = block_sum(sb, red);
        ra = 1.f / sqrtf(sa / (float)W + eps);
        rb = 1.f / sqrtf(sb / (float)W + eps);
    }
    __syncthreads();
    float ss = 0.f;
    for (int c = tid * VEC; c < W; c += HC_THREADS * VEC) {
        float x[SMAX][VEC];
#pragma unroll
        for (int s = 0; s < SMAX; ++s) {
            if (s < S) {
                ldv<VEC>(xr + (long long)s * W + c, x[s]);
            } else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) x[s][i] = 0.f;
            }
        }
        if (ar != nullptr) {
            float y[VEC];
            ldv<VEC>(ar + c, y);
            if (br != nullptr) {
                float y2[VEC], w1[VEC], w2[VEC];
                ldv<VEC>(br + c, y2);
                ldv<VEC>(wa + c, w1);
                ldv<VEC>(wb + c, w2);
#pragma unroll
                for (int i = 0; i < VEC; ++i) y[i] = 0.5f * (y[i] * ra * w1[i] + y2[i] * rb * w2[i]);
            }
            float nx[SMAX][VEC];
#pragma unroll
            for (int t = 0; t < SMAX; ++t) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) nx[t][i] = 0.f;
                if (t < S) {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) nx[t][i] = co[t] * y[i];
#pragma unroll
                    for (int s = 0; s < SMAX; ++s)
                        if (s < S) {
                            const float m = cm[s * S + t];
#pragma unroll
                            for (int i = 0; i < VEC; ++i) nx[t][i] = fmaf(m, x[s][i], nx[t][i]);
                        }
                    stv<VEC>(xr + (long long)t * W + c, nx[t]);
                }
            }
#pragma unroll
            for (int t = 0; t < SMAX; ++t)
#pragma unroll
                for (int i = 0; i < VEC; ++i) x[t][i] = nx[t][i];
        }
        if (inw != nullptr) {
            float u[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) u[i] = 0.f;
#pragma unroll
            for (int s = 0; s < SMAX; ++s)
                if (s < S) {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) u[i] = fmaf(ci[s], x[s][i], u[i]);
                }
            stv<VEC>(us + c, u);
#pragma unroll
            for (int i = 0; i < VEC; ++i) ss = fmaf(u[i], u[i], ss);
        }
    }
    if (inw == nullptr) return;
    ss = block_sum(ss, red);
    const float r = 1.f / sqrtf(ss / (float)W + eps);
    for (int c = tid * VEC; c < W; c += HC_THREADS * VEC) {
        float u[VEC], w[VEC];
        ldv<VEC>(us + c, u);
        ldv<VEC>(wn + c, w);
#pragma unroll
        for (int i = 0; i < VEC; ++i) u[i] = u[i] * r * w[i];
        stv<VEC>(h + n * W + c, u);
    }
}

}  // namespace

// X [N, S, W] fp32, updated in place when ya != NULL (the write of a sublayer whose output is ya, or -- with yb -- the
// mean of the two normed branches ya, yb with weights wa, wb [W]); mix [S, S] is indexed [from, to], outw [S].
// With inw != NULL the read of the next sublayer follows: h [N, W] = RMS norm (weight wn [W]) of sum_s inw[s] x_s.
// y_dtype (ya, yb) and h_dtype: 0 = bf16, 1 = fp32.
NXD_API int nxd_hc_step(int y_dtype, int h_dtype, float* X, const void* ya, const void* yb, const float* wa,
                        const float* wb, const float* mix, const float* outw, const float* inw, const float* wn, void* h,
                        long long N, int S, int W, float eps, void* stream) {
    if (N == 0) return 0;
    NXD_REQUIRE(S >= 1 && S <= HC_MAX, "hyper-connections: %d streams (at most %d)", S, HC_MAX);
    NXD_REQUIRE(ya == nullptr || (mix != nullptr && outw != nullptr), "hyper-connections: write without %s", "weights");
    NXD_REQUIRE(yb == nullptr || (ya != nullptr && wa != nullptr && wb != nullptr), "hyper-connections: second branch without %s", "the first");
    NXD_REQUIRE(inw == nullptr || (wn != nullptr && h != nullptr), "hyper-connections: read without %s", "norm weight");
    NXD_REQUIRE(N < (1ll << 31), "hyper-connections: %lld tokens", N);
    const size_t smem = (size_t)W * sizeof(float);
    NXD_REQUIRE(smem <= 200 * 1024, "hyper-connections: width %d", W);
    cudaStream_t st = (cudaStream_t)stream;
    auto al = [](const void* p) { return p == nullptr || ((uintptr_t)p % 16) == 0; };
    const bool vec = W % 4 == 0 && S <= 4 && al(X) && al(ya) && al(yb) && al(wa) && al(wb) && al(wn) && al(h);
#define NXD_HC_K(TY, TH, SM, V)                                                                                       \
    do {                                                                                                              \
        auto kern = hc_step_kernel<TY, TH, SM, V>;                                                                    \
        if (smem > 48 * 1024)                                                                                         \
            NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));       \
        kern<<<(unsigned)N, HC_THREADS, smem, st>>>(X, (const TY*)ya, (const TY*)yb, wa, wb, mix, outw, inw, wn, (TH*)h, S, \
                                                    W, eps);                                                          \
    } while (0)
#define NXD_HC(TY, TH)                                                                                                \
    do {                                                                                                              \
        if (vec && S <= 2) NXD_HC_K(TY, TH, 2, 4);                                                                    \
        else if (vec) NXD_HC_K(TY, TH, 4, 4);                                                                         \
        else NXD_HC_K(TY, TH, HC_MAX, 1);                                                                             \
    } while (0)
    if (y_dtype == 0 && h_dtype == 0) NXD_HC(bf16, bf16);
    else if (y_dtype == 1 && h_dtype == 0) NXD_HC(float, bf16);
    else if (y_dtype == 1 && h_dtype == 1) NXD_HC(float, float);
    else NXD_REQUIRE(false, "hyper-connections: dtypes %d -> %d", y_dtype, h_dtype);
#undef NXD_HC_K
#undef NXD_HC
    NXD_LAUNCH_CHECK();
    return 0;
}
