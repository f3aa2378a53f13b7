// Gated delta rule: a recurrent mixer whose per-head state S [D, Dv] (fp32, one per cache line) is decayed, corrected by
// the error of its own prediction and read out, token by token:
//
//     S <- g_t * S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//
// g_t is one number per head, or one per head and key channel (it then scales the rows of S).  Queries, keys and values
// come out of a short causal convolution over time (per channel, no bias) followed by silu; queries and keys are then
// unit vectors per head (the queries also scaled).  Three kernels:
//
//   delta_prep         convolution + silu (+ unit norm) of the step's q | k | v channels -> fp32; tokens before the step
//                      come from the line's convolution state (the last taps - 1 raw projections), zeros before the
//                      start of the sequence
//   delta_conv_state   moves the convolution state to the end of the step
//   delta_scan         the recurrence.  The columns of S are independent, so a thread owns a slice of one column in
//                      registers (R lanes share a column and split its rows); the step's tokens stream through shared
//                      memory in blocks, where decays (exp(-exp(A) softplus(a + bias))) and beta (sigmoid) are computed
//                      in fp32 from the pre-activations.  Per token both dot products are taken against the decayed
//                      state in one pass, o = (gS)^T q + u (k . q), then the rank-one update.  A row that starts at
//                      position 0 starts from the zero state, any other row continues from its line's state; padding
//                      tokens (t >= n_new[b]) change nothing and come out as zeros.
// This file is compiled without fast-math: the state lives for thousands of steps.
#include "common.cuh"

namespace {

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

constexpr int MAX_TAPS = 16;

// raw projection of channel `c` (column `col` of the row) at step index s (may be negative: before the step)
template <typename T>
__device__ __forceinline__ float conv_input(const T* __restrict__ proj, long long ld, const float* __restrict__ state,
                                            long long row0, int s, int p0, int K, int C, int c, long long col) {
    if (s >= 0) return ldf(proj + (row0 + s) * ld + col);
    if (p0 + s < 0) return 0.f;                                  // before the start of the sequence
    return state[(long long)(K + s) * C + c];                    // slot K + s holds position p0 + s
}

template <typename T>
__global__ void delta_prep_kernel(const T* __restrict__ proj, long long ld, int off_q, int off_k, int off_v,
                                  const float* __restrict__ conv_w, const float* __restrict__ conv_state,
                                  float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ vn,
                                  const int* __restrict__ q_start, const int* __restrict__ n_new,
                                  const int* __restrict__ seq_ids, long long units, int Tn, int H, int G, int D, int Dv,
                                  int taps, float qscale, float unit_eps) {
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= units) return;
    const int per_row = 2 * G + H;
    const long long n = unit / per_row;
    const int u = (int)(unit % per_row);
    const int b = (int)(n / Tn), t = (int)(n % Tn);
    if (n_new != nullptr && t >= n_new[b]) return;
    const int C = 2 * G * D + H * Dv, K = taps - 1;
    int cbase, dim;
    long long col;
    float* dst;
    bool unitnorm;
    float mul = 1.f;
    if (u < G) {
        cbase = u * D, col = off_q + (long long)u * D, dim = D, dst = qn + (n * G + u) * D, unitnorm = true, mul = qscale;
    } else if (u < 2 * G) {
        cbase = G * D + (u - G) * D, col = off_k + (long long)(u - G) * D, dim = D, dst = kn + (n * G + (u - G)) * D;
        unitnorm = true;
    } else {
        cbase = 2 * G * D + (u - 2 * G) * Dv, col = off_v + (long long)(u - 2 * G) * Dv, dim = Dv;
        dst = vn + (n * H + (u - 2 * G)) * Dv, unitnorm = false;
    }
    const int line = seq_ids != nullptr ? seq_ids[b] : b;
    const int p0 = q_start[b];
    const float* st = conv_state + (long long)line * K * C;
    const long long row0 = (long long)b * Tn;
    float ss = 0.f;
    for (int i = lane; i < dim; i += 32) {
        const float* w = conv_w + (long long)(cbase + i) * taps;
        float acc = 0.f;
        for (int j = 0; j < taps; ++j)
            acc = fmaf(w[j], conv_input(proj, ld, st, row0, t - (K - j), p0, K, C, cbase + i, col + i), acc);
        const float v = silu_f(acc);
        dst[i] = v;
        ss = fmaf(v, v, ss);
    }
    if (!unitnorm) return;
    ss = warp_sum(ss);
    const float r = mul / sqrtf(ss + unit_eps);
    for (int i = lane; i < dim; i += 32) dst[i] *= r;            // every lane rescales what it wrote itself
}

template <typename T>
__global__ void delta_conv_state_kernel(const T* __restrict__ proj, long long ld, int off_q, int off_k, int off_v,
                                        float* __restrict__ conv_state, const int* __restrict__ q_start,
                                        const int* __restrict__ n_new, const int* __restrict__ seq_ids, int B, int Tn,
                                        int GD, int C, int taps) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)B * C) return;
    const int b = (int)(idx / C), c = (int)(idx % C);
    const int n = n_new != nullptr ? min(n_new[b], Tn) : Tn;
    if (n <= 0) return;
    const int K = taps - 1;
    const int line = seq_ids != nullptr ? seq_ids[b] : b;
    const int p0 = q_start[b];
    const long long col = c < GD ? off_q + c : (c < 2 * GD ? off_k + (c - GD) : off_v + (c - 2 * GD));
    float* st = conv_state + (long long)line * K * C;
    float vals[MAX_TAPS];
    for (int s = 0; s < K; ++s)                                  // slot s <- position (p0 + n) - K + s
        vals[s] = conv_input(proj, ld, st, (long long)b * Tn, n - K + s, p0, K, C, c, col);
    for (int s = 0; s < K; ++s) st[(long long)s * C + c] = vals[s];
}

constexpr int SCAN_THREADS = 128, SCAN_TS = 16;

template <int NPT>
__global__ void __launch_bounds__(SCAN_THREADS)
delta_scan_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vn,
                  const float* __restrict__ apre, long long ld_a, int a_off, const float* __restrict__ bpre,
                  long long ld_b, int b_off, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                  float* __restrict__ S, float* __restrict__ out, const int* __restrict__ q_start,
                  const int* __restrict__ n_new, const int* __restrict__ seq_ids, int Tn, int H, int G, int D, int Dv,
                  int per_channel, int R) {
    extern __shared__ float smem[];
    const int Dpad = R * NPT, CT = SCAN_THREADS / R, cpw = 32 / R;      // columns per block / per warp
    float* ks = smem;                                  // [TS][Dpad]
    float* qs = ks + SCAN_TS * Dpad;                   // [TS][Dpad]
    float* gs = qs + SCAN_TS * Dpad;                   // [TS][Dpad] (per channel) or [TS]
    float* vs = gs + (per_channel ? SCAN_TS * Dpad : SCAN_TS);          // [TS][CT]
    float* bs = vs + SCAN_TS * CT;                     // [TS] beta
    float* kq = bs + SCAN_TS;                          // [TS] k . q
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = lane / cpw, cl = lane % cpw;
    const int col0 = blockIdx.x * CT, col = col0 + warp * cpw + cl;
    const int h = blockIdx.y, b = blockIdx.z, kvh = h / (H / G);
    const int n = n_new != nullptr ? min(n_new[b], Tn) : Tn;
    const long long row0 = (long long)b * Tn;
    float* orow = out + (row0 * H + h) * Dv;           // + t * H * Dv + col
    if (r == 0 && col < Dv)
        for (int t = max(n, 0); t < Tn; ++t) orow[(long long)t * H * Dv + col] = 0.f;
    if (n <= 0) return;
    const int line = seq_ids != nullptr ? seq_ids[b] : b;
    float* Sb = S + ((long long)line * H + h) * D * Dv;
    float s[NPT];
    const bool fresh = q_start[b] == 0;
#pragma unroll
    for (int ii = 0; ii < NPT; ++ii) {
        const int i = r * NPT + ii;
        s[ii] = (!fresh && i < D && col < Dv) ? Sb[(long long)i * Dv + col] : 0.f;
    }
    const float decay_rate = expf(a_log[h]);
    for (int t0 = 0; t0 < n; t0 += SCAN_TS) {
        const int cnt = min(SCAN_TS, n - t0);
        __syncthreads();
        for (int idx = tid; idx < cnt * Dpad; idx += SCAN_THREADS) {
            const int tt = idx / Dpad, i = idx - tt * Dpad;
            const long long row = row0 + t0 + tt;
            float kv = 0.f, qv = 0.f, gv = 1.f;
            if (i < D) {
                kv = kn[(row * G + kvh) * D + i];
                qv = qn[(row * G + kvh) * D + i];
                if (per_channel)
                    gv = expf(-decay_rate * softplus_f(apre[row * ld_a + a_off + (long long)h * D + i] + dt_bias[h * D + i]));
            }
            ks[idx] = kv;
            qs[idx] = qv;
            if (per_channel) gs[idx] = gv;
        }
        for (int idx = tid; idx < cnt * CT; idx += SCAN_THREADS) {
            const int tt = idx / CT, c = idx - tt * CT;
            vs[idx] = col0 + c < Dv ? vn[((row0 + t0 + tt) * H + h) * Dv + col0 + c] : 0.f;
        }
        if (tid < cnt) {
            const long long row = row0 + t0 + tid;
            bs[tid] = 1.f / (1.f + expf(-bpre[row * ld_b + b_off + h]));
            if (!per_channel) gs[tid] = expf(-decay_rate * softplus_f(apre[row * ld_a + a_off + h] + dt_bias[h]));
        }
        __syncthreads();
        for (int tt = warp; tt < cnt; tt += SCAN_THREADS / 32) {
            float d = 0.f;
            for (int i = lane; i < D; i += 32) d = fmaf(ks[tt * Dpad + i], qs[tt * Dpad + i], d);
            d = warp_sum(d);
            if (lane == 0) kq[tt] = d;
        }
        __syncthreads();
        for (int tt = 0; tt < cnt; ++tt) {
            const float* kk = ks + tt * Dpad + r * NPT;
            const float* qq = qs + tt * Dpad + r * NPT;
            float d1 = 0.f, d2 = 0.f;
            if (per_channel) {
                const float* gg = gs + tt * Dpad + r * NPT;
#pragma unroll
                for (int ii = 0; ii < NPT; ++ii) {
                    s[ii] *= gg[ii];
                    d1 = fmaf(s[ii], kk[ii], d1);
                    d2 = fmaf(s[ii], qq[ii], d2);
                }
            } else {
                const float g = gs[tt];
#pragma unroll
                for (int ii = 0; ii < NPT; ++ii) {
                    s[ii] *= g;
                    d1 = fmaf(s[ii], kk[ii], d1);
                    d2 = fmaf(s[ii], qq[ii], d2);
                }
            }
            for (int off = cpw; off < 32; off <<= 1) {
                d1 += __shfl_xor_sync(0xffffffffu, d1, off);
                d2 += __shfl_xor_sync(0xffffffffu, d2, off);
            }
            const float u = bs[tt] * (vs[tt * CT + warp * cpw + cl] - d1);
#pragma unroll
            for (int ii = 0; ii < NPT; ++ii) s[ii] = fmaf(kk[ii], u, s[ii]);
            if (r == 0 && col < Dv) orow[(long long)(t0 + tt) * H * Dv + col] = fmaf(u, kq[tt], d2);
        }
    }
    if (col < Dv) {
#pragma unroll
        for (int ii = 0; ii < NPT; ++ii) {
            const int i = r * NPT + ii;
            if (i < D) Sb[(long long)i * Dv + col] = s[ii];
        }
    }
}

template <int NPT>
int launch_scan(const float* qn, const float* kn, const float* vn, const float* apre, long long ld_a, int a_off,
                const float* bpre, long long ld_b, int b_off, const float* a_log, const float* dt_bias, float* S,
                float* out, const int* q_start, const int* n_new, const int* seq_ids, int B, int Tn, int H, int G, int D,
                int Dv, int per_channel, int R, cudaStream_t st) {
    const int Dpad = R * NPT, CT = SCAN_THREADS / R;
    const size_t smem = (size_t)(SCAN_TS * Dpad * (per_channel ? 3 : 2) + (per_channel ? 0 : SCAN_TS) + SCAN_TS * CT +
                                 2 * SCAN_TS) * sizeof(float);
    auto kern = delta_scan_kernel<NPT>;
    if (smem > 48 * 1024) NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((Dv + CT - 1) / CT, H, B);
    kern<<<grid, SCAN_THREADS, smem, st>>>(qn, kn, vn, apre, ld_a, a_off, bpre, ld_b, b_off, a_log, dt_bias, S, out,
                                           q_start, n_new, seq_ids, Tn, H, G, D, Dv, per_channel, R);
    NXD_LAUNCH_CHECK();
    return 0;
}

}  // namespace

// dtype of proj: 0 bf16, 1 fp32.  proj [B * Tn, ld]: raw q (G * D channels) at column off_q, k (G * D) at off_k, v
// (H * Dv) at off_v.  conv_w fp32 [2 G D + H Dv, taps] in q | k | v order, last column = the current token.  conv_state fp32
// [lines, taps - 1, C]: the last raw projections of every line (read here, moved on by nxd_delta_conv_state).
// qn, kn [B * Tn, G, D], vn [B * Tn, H, Dv] fp32: silu(conv), queries and keys divided by sqrt(sum x^2 + unit_eps), queries
// times qscale.  q_start [B], n_new [B] or NULL, seq_ids [B] or NULL as in the attention entry points.
NXD_API int nxd_delta_prep(int dtype, const void* proj, long long ld, int off_q, int off_k, int off_v, const float* conv_w,
                           const float* conv_state, float* qn, float* kn, float* vn, const int* q_start, const int* n_new,
                           const int* seq_ids, int B, int Tn, int H, int G, int D, int Dv, int taps, float qscale,
                           float unit_eps, void* stream) {
    const long long units = (long long)B * Tn * (2 * G + H);
    if (units == 0) return 0;
    NXD_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "short convolution with %d taps", taps);
    const int wpb = 8;
    const unsigned blocks = (unsigned)((units + wpb - 1) / wpb);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == 0)
        delta_prep_kernel<bf16><<<blocks, wpb * 32, 0, st>>>((const bf16*)proj, ld, off_q, off_k, off_v, conv_w, conv_state, qn,
                                                            kn, vn, q_start, n_new, seq_ids, units, Tn, H, G, D, Dv, taps,
                                                            qscale, unit_eps);
    else
        delta_prep_kernel<float><<<blocks, wpb * 32, 0, st>>>((const float*)proj, ld, off_q, off_k, off_v, conv_w, conv_state,
                                                             qn, kn, vn, q_start, n_new, seq_ids, units, Tn, H, G, D, Dv,
                                                             taps, qscale, unit_eps);
    NXD_LAUNCH_CHECK();
    return 0;
}

// After nxd_delta_prep of the same step: slot s of the line's state <- raw projection of position end - (taps - 1) + s,
// end = q_start + n_new (zeros before the start of the sequence).  Rows without real tokens keep their state.
NXD_API int nxd_delta_conv_state(int dtype, const void* proj, long long ld, int off_q, int off_k, int off_v,
                                 float* conv_state, const int* q_start, const int* n_new, const int* seq_ids, int B, int Tn,
                                 int H, int G, int D, int Dv, int taps, void* stream) {
    const int C = 2 * G * D + H * Dv;
    if ((long long)B * C == 0 || taps <= 1) return 0;
    NXD_REQUIRE(taps <= MAX_TAPS, "short convolution with %d taps", taps);
    const unsigned blocks = (unsigned)(((long long)B * C + 255) / 256);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == 0)
        delta_conv_state_kernel<bf16><<<blocks, 256, 0, st>>>((const bf16*)proj, ld, off_q, off_k, off_v, conv_state, q_start,
                                                             n_new, seq_ids, B, Tn, G * D, C, taps);
    else
        delta_conv_state_kernel<float><<<blocks, 256, 0, st>>>((const float*)proj, ld, off_q, off_k, off_v, conv_state,
                                                              q_start, n_new, seq_ids, B, Tn, G * D, C, taps);
    NXD_LAUNCH_CHECK();
    return 0;
}

// qn, kn, vn as written by nxd_delta_prep.  apre fp32 [B * Tn, ld_a]: decay pre-activation of head h at column a_off + h
// (per_channel == 0) or of (h, key channel i) at a_off + h * D + i; dt_bias [H] or [H * D], a_log [H]:
// g = exp(-exp(a_log) softplus(apre + dt_bias)).  bpre fp32 [B * Tn, ld_b]: beta = sigmoid(bpre[b_off + h]).
// S fp32 [lines, H, D, Dv], updated in place.  out fp32 [B * Tn, H, Dv].
NXD_API int nxd_delta_scan(const float* qn, const float* kn, const float* vn, const float* apre, long long ld_a, int a_off,
                           const float* bpre, long long ld_b, int b_off, const float* a_log, const float* dt_bias, float* S,
                           float* out, const int* q_start, const int* n_new, const int* seq_ids, int B, int Tn, int H, int G,
                           int D, int Dv, int per_channel, void* stream) {
    if ((long long)B * Tn * H * Dv == 0) return 0;
    NXD_REQUIRE(G > 0 && H % G == 0, "delta rule: %d heads over %d query/key heads", H, G);
    NXD_REQUIRE(D >= 1 && D <= 1024, "delta rule: key size %d", D);
    cudaStream_t st = (cudaStream_t)stream;
    // rows of a column per thread (NPT) and lanes per column (R, a power of two): the smallest slice that keeps R <= 4,
    // wider keys spread over more lanes
    const int npt = D <= 32 ? 8 : (D <= 64 ? 16 : 32);
    int R = 1;
    while (R * npt < D) R <<= 1;
#define NXD_SCAN(N)                                                                                                      \
    return launch_scan<N>(qn, kn, vn, apre, ld_a, a_off, bpre, ld_b, b_off, a_log, dt_bias, S, out, q_start, n_new,       \
                          seq_ids, B, Tn, H, G, D, Dv, per_channel, R, st)
    if (npt == 8) NXD_SCAN(8);
    if (npt == 16) NXD_SCAN(16);
    NXD_SCAN(32);
#undef NXD_SCAN
}
