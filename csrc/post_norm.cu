// RMS norm with a zero-centred weight, applied to a sublayer's OUTPUT and added to an fp32 residual stream:
//
//   n = y / sqrt(mean(y^2) + eps) * (1 + w);   x <- x + n  (x fp32, in place);   h = cast(x)   (optional)
//
// With x == NULL the kernel is the plain norm (h = cast(n)): the model's final norm.  One CTA per row, the row is read
// once into registers (up to 16 values per thread, above that it is re-read), statistics in fp32.
#include "common.cuh"

namespace {

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int PN_THREADS = 128, PN_REG = 16;

template <typename TY, typename TW, typename TH>
__global__ void __launch_bounds__(PN_THREADS)
post_norm_kernel(const TY* __restrict__ y, const TW* __restrict__ w, float* __restrict__ x, TH* __restrict__ h, int W,
                 float eps, float offset) {
    __shared__ float red[32];
    const long long row = blockIdx.x;
    const TY* yr = y + row * W;
    float v[PN_REG];
    float ss = 0.f;
    const bool in_regs = W <= PN_REG * PN_THREADS;
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < PN_REG; ++i) {
            const int c = threadIdx.x + i * PN_THREADS;
            v[i] = c < W ? ldf(yr + c) : 0.f;
            ss += v[i] * v[i];
        }
    } else {
        for (int c = threadIdx.x; c < W; c += PN_THREADS) {
            const float t = ldf(yr + c);
            ss += t * t;
        }
    }
    ss = block_sum(ss, red);
    const float r = 1.f / sqrtf(ss / (float)W + eps);
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < PN_REG; ++i) {
            const int c = threadIdx.x + i * PN_THREADS;
            if (c < W) {
                float n = v[i] * r * (offset + ldf(w + c));
                if (x != nullptr) {
                    n += x[row * W + c];
                    x[row * W + c] = n;
                }
                if (h != nullptr) stf(h + row * W + c, n);
            }
        }
    } else {
        for (int c = threadIdx.x; c < W; c += PN_THREADS) {
            float n = ldf(yr + c) * r * (offset + ldf(w + c));
            if (x != nullptr) {
                n += x[row * W + c];
                x[row * W + c] = n;
            }
            if (h != nullptr) stf(h + row * W + c, n);
        }
    }
}

template <typename TY, typename TW, typename TH>
int launch(const void* y, const void* w, float* x, void* h, long long rows, int W, float eps, float offset,
           cudaStream_t st) {
    post_norm_kernel<TY, TW, TH><<<(unsigned)rows, PN_THREADS, 0, st>>>((const TY*)y, (const TW*)w, x, (TH*)h, W, eps,
                                                                        offset);
    NXD_LAUNCH_CHECK();
    return 0;
}


// Pre- and post-norm of one sublayer boundary in a single pass over an fp32 residual stream:
//
//   (y given)       x <- x + norm(y) * w_post                  (norm on the sublayer's output, x in place)
//   (w_next given)  h  = cast(norm(x) * w_next)                (the next sublayer's input)
//
// norm(v) = (v - mean(v)) / sqrt(var(v) + eps) with center != 0 (layer norm, weight only), v / sqrt(mean(v^2) + eps)
// otherwise.  One CTA per row; the row sits in shared memory, mean and variance are two separate fp32 reductions.
template <typename TY, typename TH>
__global__ void __launch_bounds__(PN_THREADS)
norm_chain_kernel(const TY* __restrict__ y, const float* __restrict__ w_post, float* __restrict__ x,
                  const float* __restrict__ w_next, TH* __restrict__ h, int W, float eps, int center) {
    extern __shared__ float rowbuf[];
    __shared__ float red[32];
    const long long row = blockIdx.x;
    float* xr = x + row * W;
    if (y != nullptr) {
        const TY* yr = y + row * W;
        float s = 0.f;
        for (int c = threadIdx.x; c < W; c += PN_THREADS) {
            const float v = ldf(yr + c);
            rowbuf[c] = v;
            s += v;
        }
        const float mean = center ? block_sum(s, red) / (float)W : 0.f;
        float ss = 0.f;
        for (int c = threadIdx.x; c < W; c += PN_THREADS) {
            const float d = rowbuf[c] - mean;
            ss += d * d;
        }
        const float r = 1.f / sqrtf(block_sum(ss, red) / (float)W + eps);
        for (int c = threadIdx.x; c < W; c += PN_THREADS) {
            const float v = xr[c] + (rowbuf[c] - mean) * r * w_post[c];
            xr[c] = v;
            rowbuf[c] = v;
        }
    } else {
        for (int c = threadIdx.x; c < W; c += PN_THREADS) rowbuf[c] = xr[c];
    }
    if (w_next == nullptr || h == nullptr) return;
    float s = 0.f;
    for (int c = threadIdx.x; c < W; c += PN_THREADS) s += rowbuf[c];
    const float mean = center ? block_sum(s, red) / (float)W : 0.f;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += PN_THREADS) {
        const float d = rowbuf[c] - mean;
        ss += d * d;
    }
    const float r = 1.f / sqrtf(block_sum(ss, red) / (float)W + eps);
    TH* hr = h + row * W;
    for (int c = threadIdx.x; c < W; c += PN_THREADS) stf(hr + c, (rowbuf[c] - mean) * r * w_next[c]);
}

template <typename TY, typename TH>
int launch_chain(const void* y, const float* w_post, float* x, const float* w_next, void* h, long long rows, int W,
                 float eps, int center, cudaStream_t st) {
    const size_t smem = (size_t)W * sizeof(float);
    auto kern = norm_chain_kernel<TY, TH>;
    if (smem > 48 * 1024) NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<(unsigned)rows, PN_THREADS, smem, st>>>((const TY*)y, w_post, x, w_next, (TH*)h, W, eps, center);
    NXD_LAUNCH_CHECK();
    return 0;
}

// Parallel sublayers with layer scale and a gated residual, and the next layer's norm, in one pass over the fp32 stream:
//
//   x <- x + ls1 * sigmoid(gate[:, off1 + c] + gb1) * y1  +  ls2 * sigmoid(gate[:, off2 + c] + gb2) * (y2 + y2b)
//   h  = cast(x / sqrt(mean(x^2) + eps) * w_next[0])            (the norm's weight is ONE number)
//
// y1 == NULL: no update (the plain norm of the stream); y2 == NULL: one sublayer; w_next == NULL: no h.
__device__ __forceinline__ float ld_any(const void* p, int is_f32, long long i) {
    return is_f32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
}

__device__ __forceinline__ void ld4_any(const void* p, int is_f32, long long i, float (&v)[4]) {
    if (is_f32) {
        const float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
        v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
    } else {
        const uint2 t = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(p) + i);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const bf162*>(&t.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const bf162*>(&t.y));
        v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
    }
}
__device__ __forceinline__ void ld4_vec(const float* p, int c, float (&v)[4]) {
    if (p == nullptr) {
        v[0] = v[1] = v[2] = v[3] = 0.f;
        return;
    }
    const float4 t = *reinterpret_cast<const float4*>(p + c);
    v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
}
__device__ __forceinline__ void st4(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void st4(bf16* p, const float (&v)[4]) {
    uint2 t;
    *reinterpret_cast<bf162*>(&t.x) = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<bf162*>(&t.y) = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = t;
}

// VEC = 4: four consecutive columns per thread and iteration through 8- / 16-byte accesses (widths, gate offsets and
// pitches that are multiples of 4); VEC = 1: any sizes.
template <typename TH, int VEC>
__global__ void __launch_bounds__(PN_THREADS)
gated_residual_norm_kernel(float* __restrict__ x, const void* __restrict__ y1, int y1_f32, const void* __restrict__ y2,
                           int y2_f32, const float* __restrict__ y2_bias, const void* __restrict__ gate, int gate_f32,
                           long long ld_g, int off1, int off2, const float* __restrict__ gb1,
                           const float* __restrict__ gb2, const float* __restrict__ ls1, const float* __restrict__ ls2,
                           const float* __restrict__ w_next, TH* __restrict__ h, int W, float eps) {
    extern __shared__ __align__(16) float rowbuf[];
    __shared__ float red[32];
    const long long row = blockIdx.x;
    float* xr = x + row * W;
    float ss = 0.f;
    if (VEC == 4) {
        for (int c = threadIdx.x * 4; c < W; c += PN_THREADS * 4) {
            float v[4];
            ld4_vec(xr, c, v);
            if (y1 != nullptr) {
                float a[4], z[4], t[4];
                ld4_any(y1, y1_f32, row * W + c, a);
                if (ls1 != nullptr) {
                    ld4_vec(ls1, c, t);
#pragma unroll
                    for (int i = 0; i < 4; ++i) a[i] *= t[i];
                }
                if (gate != nullptr) {
                    ld4_any(gate, gate_f32, row * ld_g + off1 + c, z);
                    ld4_vec(gb1, c, t);
#pragma unroll
                    for (int i = 0; i < 4; ++i) a[i] *= 1.f / (1.f + expf(-(z[i] + t[i])));
                }
                if (y2 != nullptr) {
                    float f[4];
                    ld4_any(y2, y2_f32, row * W + c, f);
                    ld4_vec(y2_bias, c, t);
#pragma unroll
                    for (int i = 0; i < 4; ++i) f[i] += t[i];
                    if (ls2 != nullptr) {
                        ld4_vec(ls2, c, t);
#pragma unroll
                        for (int i = 0; i < 4; ++i) f[i] *= t[i];
                    }
                    if (gate != nullptr) {
                        ld4_any(gate, gate_f32, row * ld_g + off2 + c, z);
                        ld4_vec(gb2, c, t);
#pragma unroll
                        for (int i = 0; i < 4; ++i) f[i] *= 1.f / (1.f + expf(-(z[i] + t[i])));
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) a[i] += f[i];
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] += a[i];
                st4(xr + c, v);
            }
            st4(rowbuf + c, v);
#pragma unroll
            for (int i = 0; i < 4; ++i) ss = fmaf(v[i], v[i], ss);
        }
    } else {
        for (int c = threadIdx.x; c < W; c += PN_THREADS) {
            float v = xr[c];
            if (y1 != nullptr) {
                float z = gate != nullptr ? ld_any(gate, gate_f32, row * ld_g + off1 + c) + (gb1 != nullptr ? gb1[c] : 0.f) : 0.f;
                float a = ld_any(y1, y1_f32, row * W + c) * (ls1 != nullptr ? ls1[c] : 1.f);
                if (gate != nullptr) a *= 1.f / (1.f + expf(-z));
                if (y2 != nullptr) {
                    float f = (ld_any(y2, y2_f32, row * W + c) + (y2_bias != nullptr ? y2_bias[c] : 0.f)) *
                              (ls2 != nullptr ? ls2[c] : 1.f);
                    if (gate != nullptr) {
                        z = ld_any(gate, gate_f32, row * ld_g + off2 + c) + (gb2 != nullptr ? gb2[c] : 0.f);
                        f *= 1.f / (1.f + expf(-z));
                    }
                    a += f;
                }
                v += a;
                xr[c] = v;
            }
            rowbuf[c] = v;
            ss = fmaf(v, v, ss);
        }
    }
    if (w_next == nullptr || h == nullptr) return;
    const float r = w_next[0] / sqrtf(block_sum(ss, red) / (float)W + eps);
    TH* hr = h + row * W;
    if (VEC == 4) {
        for (int c = threadIdx.x * 4; c < W; c += PN_THREADS * 4) {
            float v[4];
            ld4_vec(rowbuf, c, v);
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] *= r;
            st4(hr + c, v);
        }
    } else {
        for (int c = threadIdx.x; c < W; c += PN_THREADS) stf(hr + c, rowbuf[c] * r);
    }
}

template <typename TH, int VEC>
int launch_gated(float* x, const void* y1, int y1_dtype, const void* y2, int y2_dtype, const float* y2_bias,
                 const void* gate, int gate_dtype, long long ld_g, int off1, int off2, const float* gb1, const float* gb2,
                 const float* ls1, const float* ls2, const float* w_next, void* h, long long rows, int W, float eps,
                 cudaStream_t st) {
    const size_t smem = (size_t)W * sizeof(float);
    auto kern = gated_residual_norm_kernel<TH, VEC>;
    if (smem > 48 * 1024) NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<(unsigned)rows, PN_THREADS, smem, st>>>(x, y1, y1_dtype, y2, y2_dtype, y2_bias, gate, gate_dtype, ld_g, off1, off2,
                                                   gb1, gb2, ls1, ls2, w_next, (TH*)h, W, eps);
    NXD_LAUNCH_CHECK();
    return 0;
}

}  // namespace

// x [rows, W] fp32 stream, updated in place when y1 is given.  y1, y2 [rows, W] (dtype codes 0 bf16 / 1 fp32; y2 may be
// NULL), y2_bias [W] fp32 or NULL.  gate [rows, ld_g] (gate_dtype) or NULL: the residual gates' pre-activations at
// columns off1 (for y1) and off2 (for y2), gb1 / gb2 [W] fp32 their biases (or NULL); ls1 / ls2 [W] fp32 layer scales
// (or NULL).  w_next: pointer to the ONE fp32 weight of the following norm (or NULL); h [rows, W] (h_dtype) or NULL.
NXD_API int nxd_gated_residual_norm(float* x, const void* y1, int y1_dtype, const void* y2, int y2_dtype,
                                    const float* y2_bias, const void* gate, int gate_dtype, long long ld_g, int off1,
                                    int off2, const float* gb1, const float* gb2, const float* ls1, const float* ls2,
                                    const float* w_next, void* h, int h_dtype, long long rows, int W, float eps,
                                    void* stream) {
    if (rows == 0) return 0;
    NXD_REQUIRE(rows < (1ll << 31), "gated residual: %lld rows", rows);
    NXD_REQUIRE((size_t)W * sizeof(float) <= 200 * 1024, "gated residual: width %d", W);
    cudaStream_t st = (cudaStream_t)stream;
    auto al = [](const void* p, size_t n) { return p == nullptr || ((uintptr_t)p % n) == 0; };
    const bool vec = W % 4 == 0 && ld_g % 4 == 0 && off1 % 4 == 0 && off2 % 4 == 0 && al(x, 16) && al(y1, 16) && al(y2, 16) &&
                     al(gate, 16) && al(h, 16) && al(y2_bias, 16) && al(gb1, 16) && al(gb2, 16) && al(ls1, 16) && al(ls2, 16);
#define NXD_GR(TH, V)                                                                                                  \
    return launch_gated<TH, V>(x, y1, y1_dtype, y2, y2_dtype, y2_bias, gate, gate_dtype, ld_g, off1, off2, gb1, gb2, ls1, \
                               ls2, w_next, h, rows, W, eps, st)
    if (h_dtype == 0) {
        if (vec) NXD_GR(bf16, 4);
        NXD_GR(bf16, 1);
    }
    if (vec) NXD_GR(float, 4);
    NXD_GR(float, 1);
#undef NXD_GR
}

// y [rows, W] (y_dtype), w [W] (w_dtype), x [rows, W] fp32 or NULL, h [rows, W] (h_dtype) or NULL; dtypes: 0 bf16,
// 1 fp32.  offset is added to the weight (1 for a weight stored around zero, 0 for a plain weight).
NXD_API int nxd_post_norm_residual(int y_dtype, int w_dtype, int h_dtype, const void* y, const void* w, float* x, void* h,
                                   long long rows, int W, float eps, float offset, void* stream) {
    if (rows == 0) return 0;
    NXD_REQUIRE(rows < (1ll << 31), "post norm: %lld rows", rows);
    cudaStream_t st = (cudaStream_t)stream;
    const int key = (y_dtype << 2) | (w_dtype << 1) | h_dtype;
    switch (key) {
        case 0: return launch<bf16, bf16, bf16>(y, w, x, h, rows, W, eps, offset, st);
        case 1: return launch<bf16, bf16, float>(y, w, x, h, rows, W, eps, offset, st);
        case 2: return launch<bf16, float, bf16>(y, w, x, h, rows, W, eps, offset, st);
        case 3: return launch<bf16, float, float>(y, w, x, h, rows, W, eps, offset, st);
        case 4: return launch<float, bf16, bf16>(y, w, x, h, rows, W, eps, offset, st);
        case 5: return launch<float, bf16, float>(y, w, x, h, rows, W, eps, offset, st);
        case 6: return launch<float, float, bf16>(y, w, x, h, rows, W, eps, offset, st);
        default: return launch<float, float, float>(y, w, x, h, rows, W, eps, offset, st);
    }
}

// x [rows, W] fp32 stream (updated in place when y is given); y [rows, W] (y_dtype) or NULL; w_post, w_next [W] fp32 (or
// NULL); h [rows, W] (h_dtype) or NULL.  center: 1 = layer norm (mean removed), 0 = RMS norm.
NXD_API int nxd_norm_chain(int y_dtype, int h_dtype, const void* y, const float* w_post, float* x, const float* w_next,
                           void* h, long long rows, int W, float eps, int center, void* stream) {
    if (rows == 0) return 0;
    NXD_REQUIRE(rows < (1ll << 31), "norm chain: %lld rows", rows);
    NXD_REQUIRE((size_t)W * sizeof(float) <= 200 * 1024, "norm chain: width %d", W);
    cudaStream_t st = (cudaStream_t)stream;
    switch ((y_dtype << 1) | h_dtype) {
        case 0: return launch_chain<bf16, bf16>(y, w_post, x, w_next, h, rows, W, eps, center, st);
        case 1: return launch_chain<bf16, float>(y, w_post, x, w_next, h, rows, W, eps, center, st);
        case 2: return launch_chain<float, bf16>(y, w_post, x, w_next, h, rows, W, eps, center, st);
        default: return launch_chain<float, float>(y, w_post, x, w_next, h, rows, W, eps, center, st);
    }
}
