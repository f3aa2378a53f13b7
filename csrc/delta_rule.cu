// Gated delta rule: a recurrent mixer whose per-head state S [D, Dv] (fp32, one per cache line) is decayed, corrected by
// the error of its own prediction and read out, token by token:
//
//     S <- g_t * S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//
// g_t is one number per head, or one per head and key channel (it then scales the rows of S).  Queries, keys and values
// come out of a short causal convolution over time (per channel, no bias) followed by silu; queries and keys are then
// unit vectors per head (the queries also scaled).  Four kernels:
//
//   delta_prep         convolution + silu (+ unit norm) of the step's q | k | v channels -> fp32; tokens before the step
//                      come from the line's convolution state (the last taps - 1 raw projections), zeros before the
//                      start of the sequence
//   delta_conv_state   moves the convolution state to the end of the step
//   delta_gates        decays exp(-exp(A) softplus(a + bias)) and beta = sigmoid(b) from the fp32 pre-activations, in
//                      place, one thread per value
//   delta_scan         the recurrence.  The columns of S are independent, so a thread owns a slice of one column in
//                      registers (R lanes share a column and split its rows); the step's tokens stream through shared
//                      memory in blocks of 16.  Per token both dot products are taken against the decayed
//                      state in one pass, o = (gS)^T q + u (k . q), then the rank-one update.  A row that starts at
//                      position 0 starts from the zero state, any other row continues from its line's state; padding
//                      tokens (t >= n_new[b]) change nothing and come out as zeros.
// This file is compiled without fast-math: the state lives for thousands of steps.
#include "common.cuh"
#include "mma_sync.cuh"

namespace {

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

constexpr int MAX_TAPS = 32;

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

// In place: a <- exp(-exp(a_log[h]) softplus(a + dt_bias)) for the decay pre-activations (per head: one column, per
// channel: D columns per head), b <- sigmoid(b) for the beta pre-activations.  One thread per value.
__global__ void delta_gates_kernel(float* __restrict__ apre, long long ld_a, int a_off, float* __restrict__ bpre,
                                   long long ld_b, int b_off, const float* __restrict__ a_log,
                                   const float* __restrict__ dt_bias, long long N, int H, int per_head) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int cols = H * per_head + H;                 // decay columns, then beta columns
    if (idx >= N * cols) return;
    const long long n = idx / cols;
    const int c = (int)(idx - n * cols);
    if (c < H * per_head) {
        float* p = apre + n * ld_a + a_off + c;
        *p = expf(-expf(a_log[c / per_head]) * softplus_f(*p + dt_bias[c]));
    } else {
        float* p = bpre + n * ld_b + b_off + (c - H * per_head);
        *p = 1.f / (1.f + expf(-*p));
    }
}

__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}

// A thread keeps NPT rows of one state column in registers; the R lanes that share a column sit cpw = 32 / R lanes apart.
// In shared memory the NPT values that a lane reads per token are padded to NPT + 4 floats, so that the R simultaneous
// 16-byte reads of a warp fall into different banks.  Blocks of TS tokens are double-buffered: with ASYNC the next block
// is fetched by cp.async (16 bytes a copy; key / value sizes and pitches that are multiples of 4) while the current one
// is consumed; otherwise by plain loads.
template <int NPT, bool ASYNC>
__global__ void __launch_bounds__(SCAN_THREADS)
delta_scan_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vn,
                  const float* __restrict__ gate, long long ld_a, int a_off, const float* __restrict__ beta,
                  long long ld_b, int b_off, float* __restrict__ S, float* __restrict__ out,
                  const int* __restrict__ q_start, const int* __restrict__ n_new, const int* __restrict__ seq_ids, int Tn,
                  int H, int G, int D, int Dv, int per_channel, int R, int TS) {
    extern __shared__ __align__(16) float smem[];
    constexpr int PITCH = NPT + 4;
    const int DS = R * PITCH, CT = SCAN_THREADS / R, cpw = 32 / R;      // floats per token; columns per block / per warp
    const int per_buf = TS * DS * (per_channel ? 3 : 2) + TS * CT + 2 * TS;
    float* kq = smem + 2 * per_buf;                    // [TS] k . q of the block being consumed
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
    const int Dpad = R * NPT;
    // buffer layout: k [TS][DS] | q [TS][DS] | (g [TS][DS]) | v [TS][CT] | g per head [TS] | beta [TS]
    auto fetch = [&](int t0, int buf) {
        float* ks = smem + buf * per_buf;
        float* qs = ks + TS * DS;
        float* gs = qs + TS * DS;
        float* vs = gs + (per_channel ? TS * DS : 0);
        float* gh = vs + TS * CT;
        float* bs = gh + TS;
        const int cnt = min(TS, n - t0);
        if (ASYNC) {
            const int c4 = Dpad / 4;                   // 16-byte pieces per token
            for (int idx = tid; idx < cnt * c4; idx += SCAN_THREADS) {
                const int tt = idx / c4, i = (idx - tt * c4) * 4;
                const long long row = row0 + t0 + tt;
                const int at = tt * DS + (i / NPT) * PITCH + (i % NPT);
                const bool ok = i < D;
                const long long src = (row * G + kvh) * D + (ok ? i : 0);
                mma::cp_async16((uint32_t)__cvta_generic_to_shared(ks + at), kn + src, ok);
                mma::cp_async16((uint32_t)__cvta_generic_to_shared(qs + at), qn + src, ok);
                if (per_channel)
                    mma::cp_async16((uint32_t)__cvta_generic_to_shared(gs + at),
                                    gate + row * ld_a + a_off + (long long)h * D + (ok ? i : 0), ok);
            }
            const int v4 = CT / 4;
            for (int idx = tid; idx < cnt * v4; idx += SCAN_THREADS) {
                const int tt = idx / v4, c = (idx - tt * v4) * 4;
                const bool ok = col0 + c < Dv;
                mma::cp_async16((uint32_t)__cvta_generic_to_shared(vs + tt * CT + c),
                                vn + ((row0 + t0 + tt) * H + h) * Dv + (ok ? col0 + c : 0), ok);
            }
            if (tid < cnt) {
                const long long row = row0 + t0 + tid;
                cp_async4((uint32_t)__cvta_generic_to_shared(bs + tid), beta + row * ld_b + b_off + h);
                if (!per_channel) cp_async4((uint32_t)__cvta_generic_to_shared(gh + tid), gate + row * ld_a + a_off + h);
            }
        } else {
            for (int idx = tid; idx < cnt * Dpad; idx += SCAN_THREADS) {
                const int tt = idx / Dpad, i = idx - tt * Dpad;
                const long long row = row0 + t0 + tt;
                float kv = 0.f, qv = 0.f, gv = 1.f;
                if (i < D) {
                    kv = kn[(row * G + kvh) * D + i];
                    qv = qn[(row * G + kvh) * D + i];
                    if (per_channel) gv = gate[row * ld_a + a_off + (long long)h * D + i];
                }
                const int at = tt * DS + (i / NPT) * PITCH + (i % NPT);
                ks[at] = kv;
                qs[at] = qv;
                if (per_channel) gs[at] = gv;
            }
            for (int idx = tid; idx < cnt * CT; idx += SCAN_THREADS) {
                const int tt = idx / CT, c = idx - tt * CT;
                vs[idx] = col0 + c < Dv ? vn[((row0 + t0 + tt) * H + h) * Dv + col0 + c] : 0.f;
            }
            if (tid < cnt) {
                const long long row = row0 + t0 + tid;
                bs[tid] = beta[row * ld_b + b_off + h];
                if (!per_channel) gh[tid] = gate[row * ld_a + a_off + h];
            }
        }
        mma::cp_async_commit();
    };
    fetch(0, 0);
    int buf = 0;
    for (int t0 = 0; t0 < n; t0 += TS, buf ^= 1) {
        const int cnt = min(TS, n - t0);
        if (t0 + TS < n) {
            fetch(t0 + TS, buf ^ 1);                   // the other buffer was released by the barrier that ended the last round
            mma::cp_async_wait<1>();
        } else {
            mma::cp_async_wait<0>();
        }
        __syncthreads();
        const float* ks = smem + buf * per_buf;
        const float* qs = ks + TS * DS;
        const float* gs = qs + TS * DS;
        const float* vs = gs + (per_channel ? TS * DS : 0);
        const float* gh = vs + TS * CT;
        const float* bs = gh + TS;
        for (int tt = warp; tt < cnt; tt += SCAN_THREADS / 32) {
            float d = 0.f;
            for (int i = lane; i < Dpad; i += 32) {
                const int at = tt * DS + (i / NPT) * PITCH + (i % NPT);
                d = fmaf(ks[at], qs[at], d);
            }
            d = warp_sum(d);
            if (lane == 0) kq[tt] = d;
        }
        __syncthreads();
        for (int tt = 0; tt < cnt; ++tt) {
            const float4* k4 = reinterpret_cast<const float4*>(ks + tt * DS + r * PITCH);
            const float4* q4 = reinterpret_cast<const float4*>(qs + tt * DS + r * PITCH);
            float kreg[NPT];
            float d1[4] = {0.f, 0.f, 0.f, 0.f}, d2[4] = {0.f, 0.f, 0.f, 0.f};      // four independent chains each
            if (per_channel) {
                const float4* g4 = reinterpret_cast<const float4*>(gs + tt * DS + r * PITCH);
#pragma unroll
                for (int v = 0; v < NPT / 4; ++v) {
                    const float4 kv = k4[v], qv = q4[v], gv = g4[v];
                    kreg[4 * v] = kv.x, kreg[4 * v + 1] = kv.y, kreg[4 * v + 2] = kv.z, kreg[4 * v + 3] = kv.w;
                    s[4 * v] *= gv.x, s[4 * v + 1] *= gv.y, s[4 * v + 2] *= gv.z, s[4 * v + 3] *= gv.w;
                    d1[0] = fmaf(s[4 * v], kv.x, d1[0]), d1[1] = fmaf(s[4 * v + 1], kv.y, d1[1]);
                    d1[2] = fmaf(s[4 * v + 2], kv.z, d1[2]), d1[3] = fmaf(s[4 * v + 3], kv.w, d1[3]);
                    d2[0] = fmaf(s[4 * v], qv.x, d2[0]), d2[1] = fmaf(s[4 * v + 1], qv.y, d2[1]);
                    d2[2] = fmaf(s[4 * v + 2], qv.z, d2[2]), d2[3] = fmaf(s[4 * v + 3], qv.w, d2[3]);
                }
            } else {
                const float g = gh[tt];
#pragma unroll
                for (int v = 0; v < NPT / 4; ++v) {
                    const float4 kv = k4[v], qv = q4[v];
                    kreg[4 * v] = kv.x, kreg[4 * v + 1] = kv.y, kreg[4 * v + 2] = kv.z, kreg[4 * v + 3] = kv.w;
                    s[4 * v] *= g, s[4 * v + 1] *= g, s[4 * v + 2] *= g, s[4 * v + 3] *= g;
                    d1[0] = fmaf(s[4 * v], kv.x, d1[0]), d1[1] = fmaf(s[4 * v + 1], kv.y, d1[1]);
                    d1[2] = fmaf(s[4 * v + 2], kv.z, d1[2]), d1[3] = fmaf(s[4 * v + 3], kv.w, d1[3]);
                    d2[0] = fmaf(s[4 * v], qv.x, d2[0]), d2[1] = fmaf(s[4 * v + 1], qv.y, d2[1]);
                    d2[2] = fmaf(s[4 * v + 2], qv.z, d2[2]), d2[3] = fmaf(s[4 * v + 3], qv.w, d2[3]);
                }
            }
            float e1 = (d1[0] + d1[1]) + (d1[2] + d1[3]), e2 = (d2[0] + d2[1]) + (d2[2] + d2[3]);
            for (int off = cpw; off < 32; off <<= 1) {
                e1 += __shfl_xor_sync(0xffffffffu, e1, off);
                e2 += __shfl_xor_sync(0xffffffffu, e2, off);
            }
            const float u = bs[tt] * (vs[tt * CT + warp * cpw + cl] - e1);
#pragma unroll
            for (int ii = 0; ii < NPT; ++ii) s[ii] = fmaf(kreg[ii], u, s[ii]);
            if (r == 0 && col < Dv) orow[(long long)(t0 + tt) * H * Dv + col] = fmaf(u, kq[tt], e2);
        }
        __syncthreads();                               // everyone is done with this buffer and with kq
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
int launch_scan(const float* qn, const float* kn, const float* vn, const float* gate, long long ld_a, int a_off,
                const float* beta, long long ld_b, int b_off, float* S, float* out, const int* q_start, const int* n_new,
                const int* seq_ids, int B, int Tn, int H, int G, int D, int Dv, int per_channel, int R, cudaStream_t st) {
    const int DS = R * (NPT + 4), CT = SCAN_THREADS / R;
    int TS = SCAN_TS;                                  // tokens per block: fewer for very wide keys (shared memory)
    auto bytes = [&](int ts) {
        return (size_t)(2 * (ts * DS * (per_channel ? 3 : 2) + ts * CT + 2 * ts) + ts) * sizeof(float);
    };
    while (TS > 1 && bytes(TS) > 100 * 1024) TS >>= 1;
    const size_t smem = bytes(TS);
    auto al = [](const void* p) { return ((uintptr_t)p % 16) == 0; };
    const bool async = D % 4 == 0 && Dv % 4 == 0 && CT % 4 == 0 && al(qn) && al(kn) && al(vn) &&
                       (!per_channel || (ld_a % 4 == 0 && a_off % 4 == 0 && al(gate)));
    dim3 grid((Dv + CT - 1) / CT, H, B);
#define NXD_LAUNCH_SCAN(A)                                                                                               \
    do {                                                                                                                 \
        auto kern = delta_scan_kernel<NPT, A>;                                                                           \
        if (smem > 32 * 1024)                                                                                            \
            NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));          \
        kern<<<grid, SCAN_THREADS, smem, st>>>(qn, kn, vn, gate, ld_a, a_off, beta, ld_b, b_off, S, out, q_start, n_new,  \
                                               seq_ids, Tn, H, G, D, Dv, per_channel, R, TS);                            \
    } while (0)
    if (async) NXD_LAUNCH_SCAN(true); else NXD_LAUNCH_SCAN(false);
#undef NXD_LAUNCH_SCAN
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
// g = exp(-exp(a_log) softplus(apre + dt_bias)).  bpre fp32 [B * Tn, ld_b]: beta = sigmoid(bpre[b_off + h]).  Both are
// OVERWRITTEN with g and beta (a first kernel, one thread per value; the recurrence then reads them).
// S fp32 [lines, H, D, Dv], updated in place.  out fp32 [B * Tn, H, Dv].
NXD_API int nxd_delta_scan(const float* qn, const float* kn, const float* vn, float* apre, long long ld_a, int a_off,
                           float* bpre, long long ld_b, int b_off, const float* a_log, const float* dt_bias, float* S,
                           float* out, const int* q_start, const int* n_new, const int* seq_ids, int B, int Tn, int H, int G,
                           int D, int Dv, int per_channel, void* stream) {
    if ((long long)B * Tn * H * Dv == 0) return 0;
    NXD_REQUIRE(G > 0 && H % G == 0, "delta rule: %d heads over %d query/key heads", H, G);
    NXD_REQUIRE(D >= 1 && D <= 1024, "delta rule: key size %d", D);
    cudaStream_t st = (cudaStream_t)stream;
    const long long N = (long long)B * Tn;
    const int per_head = per_channel ? D : 1;
    const long long vals = N * ((long long)H * per_head + H);
    delta_gates_kernel<<<(unsigned)((vals + 255) / 256), 256, 0, st>>>(apre, ld_a, a_off, bpre, ld_b, b_off, a_log, dt_bias,
                                                                      N, H, per_head);
    NXD_LAUNCH_CHECK();
    // rows of a column per thread (NPT) and lanes per column (R, a power of two): the smallest slice that keeps R <= 4,
    // wider keys spread over more lanes (measured at 8 heads of 256 x 512, 2 x 4096 tokens: slices of 32 / 16 / 8 rows take
    // 4.5 / 7.8 / 13.8 ms -- fewer columns per CTA re-read the keys and queries more often)
    const int npt = D <= 32 ? 8 : (D <= 64 ? 16 : 32);
    int R = 1;
    while (R * npt < D) R <<= 1;
#define NXD_SCAN(N_)                                                                                                     \
    return launch_scan<N_>(qn, kn, vn, apre, ld_a, a_off, bpre, ld_b, b_off, S, out, q_start, n_new, seq_ids, B, Tn, H, G, \
                           D, Dv, per_channel, R, st)
    if (npt == 8) NXD_SCAN(8);
    if (npt == 16) NXD_SCAN(16);
    NXD_SCAN(32);
#undef NXD_SCAN
}
