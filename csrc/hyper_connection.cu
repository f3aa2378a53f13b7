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
// streams are read once and written once, the weighted sum stays in shared memory between the two passes of the norm.
// Everything is fp32; this file is compiled without fast-math.
#include "common.cuh"

namespace {

constexpr int HC_MAX = 8, HC_THREADS = 256;

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename TY, typename TH>
__global__ void __launch_bounds__(HC_THREADS)
hc_step_kernel(float* __restrict__ X, const TY* __restrict__ ya, const TY* __restrict__ yb, const float* __restrict__ wa,
               const float* __restrict__ wb, const float* __restrict__ mix, const float* __restrict__ outw,
               const float* __restrict__ inw, const float* __restrict__ wn, TH* __restrict__ h, int S, int W, float eps) {
    extern __shared__ float us[];                  // [W] the weighted sum of the (new) streams
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
        for (int c = tid; c < W; c += HC_THREADS) {
            const float a = ldf(ar + c), b = ldf(br + c);
            sa = fmaf(a, a, sa);
            sb = fmaf(b, b, sb);
        }
        sa = block_sum(sa, red);
        sb = block_sum(sb, red);
        ra = 1.f / sqrtf(sa / (float)W + eps);
        rb = 1.f / sqrtf(sb / (float)W + eps);
    }
    __syncthreads();
    float ss = 0.f;
    for (int c = tid; c < W; c += HC_THREADS) {
        float x[HC_MAX];
#pragma unroll
        for (int s = 0; s < HC_MAX; ++s) x[s] = s < S ? xr[(long long)s * W + c] : 0.f;
        if (ar != nullptr) {
            float y = ldf(ar + c);
            if (br != nullptr) y = 0.5f * (y * ra * wa[c] + ldf(br + c) * rb * wb[c]);
            float nx[HC_MAX];
#pragma unroll
            for (int t = 0; t < HC_MAX; ++t) {
                float acc = 0.f;
                if (t < S) {
                    acc = co[t] * y;
#pragma unroll
                    for (int s = 0; s < HC_MAX; ++s)
                        if (s < S) acc = fmaf(cm[s * S + t], x[s], acc);
                    xr[(long long)t * W + c] = acc;
                }
                nx[t] = acc;
            }
#pragma unroll
            for (int t = 0; t < HC_MAX; ++t) x[t] = nx[t];
        }
        if (inw != nullptr) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < HC_MAX; ++s)
                if (s < S) u = fmaf(ci[s], x[s], u);
            us[c] = u;
            ss = fmaf(u, u, ss);
        }
    }
    if (inw == nullptr) return;
    ss = block_sum(ss, red);
    const float r = 1.f / sqrtf(ss / (float)W + eps);
    for (int c = tid; c < W; c += HC_THREADS) stf(h + n * W + c, us[c] * r * wn[c]);
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
#define NXD_HC(TY, TH)                                                                                                \
    do {                                                                                                              \
        auto kern = hc_step_kernel<TY, TH>;                                                                           \
        if (smem > 48 * 1024)                                                                                         \
            NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));       \
        kern<<<(unsigned)N, HC_THREADS, smem, st>>>(X, (const TY*)ya, (const TY*)yb, wa, wb, mix, outw, inw, wn, (TH*)h, S, \
                                                    W, eps);                                                          \
    } while (0)
    if (y_dtype == 0 && h_dtype == 0) NXD_HC(bf16, bf16);
    else if (y_dtype == 1 && h_dtype == 0) NXD_HC(float, bf16);
    else if (y_dtype == 1 && h_dtype == 1) NXD_HC(float, float);
    else NXD_REQUIRE(false, "hyper-connections: dtypes %d -> %d", y_dtype, h_dtype);
#undef NXD_HC
    NXD_LAUNCH_CHECK();
    return 0;
}
