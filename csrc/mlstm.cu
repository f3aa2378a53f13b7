// Matrix-memory recurrent mixer (mLSTM) over a per-sequence state that lives in fp32 device memory.
//
// Per head, with log-space gates i_t (input) and f_t (forget) and a running maximum m (m_0 = 0, S_0 = 0, n_0 = 0):
//
//   m_t = max(f_t + m_{t-1}, i_t)
//   S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T            S: [D, Dv]
//   n_t = exp(f_t + m_{t-1} - m_t) n_{t-1} + exp(i_t - m_t) k_t                  n: [D]
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)                       q_t already carries qscale
//
// Kernels (all statistics, gates and the state in fp32; this file is compiled without fast-math):
//   mlstm_gates       gate pre-activations as fp32 dot products of the (bf16 or fp32) mixer input with the gate rows,
//                     plus bias, soft-capped (cap * tanh(x / cap)); the forget gate goes through log-sigmoid
//   mlstm_scan        one CTA per (value-column slice, head, batch row): the slice S[:, v0 : v0 + 32] stays in
//                     registers (4 lanes per column, each holding every 4th row), the step's tokens stream through
//                     shared memory in blocks of 16; a row that starts at position 0 starts from the zero state, any
//                     other row continues from the state of its line; padding tokens (t >= n_new[b]) change nothing
//   head_norm_gate    o -> o / rms_head(o) * weight * sigmoid(gate) (unit norm and weight optional; the gate may also
//                     be silu(gate)): the output side of
//                     the recurrent mixer, and the plain output gate of an attention mixer
//   relu_squared      max(x, 0)^2
#include "common.cuh"

namespace {

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float soft_cap(float x, float cap) { return cap > 0.f ? cap * tanhf(x / cap) : x; }
__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// h [N, W], w [2 * H, W] (rows 0 .. H-1 input gate, H .. 2H-1 forget gate), bias [2 * H] fp32 -> gi, gf [N, H] fp32
template <typename T>
__global__ void mlstm_gates_kernel(const T* __restrict__ h, const T* __restrict__ w, const float* __restrict__ bias,
                                   float* __restrict__ gi, float* __restrict__ gf, long long units, int W, int H,
                                   float cap) {
    // one warp per token: the input row is read once (held in registers in pieces of 32 * GX values), the 2 * H gate
    // rows come from L1 / L2
    constexpr int GX = 8;
    const int lane = threadIdx.x & 31;
    const long long n = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= units) return;
    const T* x = h + n * W;
    for (int r0 = 0; r0 < 2 * H; r0 += 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int c0 = 0; c0 < W; c0 += 32 * GX) {
            float xv[GX];
#pragma unroll
            for (int j = 0; j < GX; ++j) {
                const int c = c0 + j * 32 + lane;
                xv[j] = c < W ? ldf(x + c) : 0.f;
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                if (r0 + r < 2 * H) {
                    const T* wr = w + (long long)(r0 + r) * W;
#pragma unroll
                    for (int j = 0; j < GX; ++j) {
                        const int c = c0 + j * 32 + lane;
                        if (c < W) acc[r] = fmaf(xv[j], ldf(wr + c), acc[r]);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const float sum = warp_sum(acc[r]);
            const int row = r0 + r;
            if (lane == 0 && row < 2 * H) {
                const float pre = soft_cap(sum + bias[row], cap);
                if (row < H) gi[n * H + row] = pre;
                else gf[n * H + row - H] = log_sigmoid(pre);
            }
        }
    }
}

constexpr int SC_THREADS = 128, SC_COLS = 32, SC_TOK = 16;

// q, k: [B * Tn, ld] rows with head hd at column q_off + hd * D (k_off + hd * D); v at v_off + hd * Dv.
// state_s [lines, H, D, Dv], state_n [lines, H, D], state_m [lines, H]; out [B * Tn, H, Dv] fp32.
template <typename T, int DPT>
__global__ void __launch_bounds__(SC_THREADS)
mlstm_scan_kernel(const T* __restrict__ proj, long long ld, int q_off, int k_off, int v_off, const float* __restrict__ gi,
                  const float* __restrict__ gf, float* __restrict__ state_s, float* __restrict__ state_n,
                  float* __restrict__ state_m, float* __restrict__ next_n, float* __restrict__ next_m,
                  float* __restrict__ out, const int* __restrict__ q_start,
                  const int* __restrict__ n_new, const int* __restrict__ seq_ids, int Tn, int H, int D, int Dv,
                  float qscale) {
    extern __shared__ float smem[];
    float* Qs = smem;                         // [SC_TOK][D]
    float* Ks = Qs + SC_TOK * D;              // [SC_TOK][D]
    float* Vs = Ks + SC_TOK * D;              // [SC_TOK][SC_COLS]
    float* Ga = Vs + SC_TOK * SC_COLS;        // [SC_TOK] decay of the old state
    float* Gb = Ga + SC_TOK;                  // [SC_TOK] weight of the new outer product
    float* Ge = Gb + SC_TOK;                  // [SC_TOK] exp(-m_t)
    float* Mx = Ge + SC_TOK;                  // [1]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int col = warp * 8 + (lane >> 2), part = lane & 3;      // 4 lanes share a value column
    const int v0 = blockIdx.x * SC_COLS, hd = blockIdx.y, b = blockIdx.z;
    const int vc = v0 + col;
    const bool col_ok = vc < Dv;
    const int nb = n_new != nullptr ? min(n_new[b], Tn) : Tn;
    const int line = seq_ids != nullptr ? seq_ids[b] : b;
    const bool fresh = q_start[b] == 0;
    float* Sg = state_s + ((long long)line * H + hd) * D * Dv;
    float* Ng = state_n + ((long long)line * H + hd) * D;
    float* Mg = state_m + (long long)line * H + hd;

    float S[DPT], nn[DPT];
#pragma unroll
    for (int r = 0; r < DPT; ++r) {
        const int d = r * 4 + part;
        const bool ok = d < D && !fresh;
        S[r] = (ok && col_ok) ? Sg[(long long)d * Dv + vc] : 0.f;
        nn[r] = ok ? Ng[d] : 0.f;
    }
    float m_run = fresh ? 0.f : *Mg;

    for (int t0 = 0; t0 < Tn; t0 += SC_TOK) {
        const int nt = min(SC_TOK, nb - t0);          // real tokens of this block (may be <= 0: only padding left)
        __syncthreads();
        if (nt > 0) {
            for (int idx = tid; idx < nt * D; idx += SC_THREADS) {
                const int t = idx / D, d = idx - t * D;
                const T* row = proj + ((long long)b * Tn + t0 + t) * ld;
                Qs[t * D + d] = ldf(row + q_off + hd * D + d) * qscale;
                Ks[t * D + d] = ldf(row + k_off + hd * D + d);
            }
            for (int idx = tid; idx < nt * SC_COLS; idx += SC_THREADS) {
                const int t = idx / SC_COLS, c = idx - t * SC_COLS;
                const T* row = proj + ((long long)b * Tn + t0 + t) * ld;
                Vs[idx] = (v0 + c < Dv) ? ldf(row + v_off + hd * Dv + v0 + c) : 0.f;
            }
            if (tid == 0) {                            // the scalar recurrence of the running maximum
                float m = m_run;
                for (int t = 0; t < nt; ++t) {
                    const long long g = ((long long)b * Tn + t0 + t) * H + hd;
                    const float f = gf[g], i = gi[g];
                    const float mn = fmaxf(f + m, i);
                    Ga[t] = expf(f + m - mn);
                    Gb[t] = expf(i - mn);
                    Ge[t] = expf(-mn);
                    m = mn;
                }
                *Mx = m;                               // the running maximum after this block, for every thread
            }
        }
        __syncthreads();
        if (nt > 0) {
            m_run = *Mx;
            for (int t = 0; t < nt; ++t) {
                const float a = Ga[t], bw = Gb[t];
                const float vt = Vs[t * SC_COLS + col] * bw;
                const float* qr = Qs + t * D;
                const float* kr = Ks + t * D;
                float num = 0.f, nq = 0.f;
#pragma unroll
                for (int r = 0; r < DPT; ++r) {
                    const int d = r * 4 + part;
                    if (d < D) {
                        const float kd = kr[d], qd = qr[d];
                        S[r] = fmaf(a, S[r], kd * vt);
                        nn[r] = fmaf(a, nn[r], bw * kd);
                        num = fmaf(S[r], qd, num);
                        nq = fmaf(nn[r], qd, nq);
                    }
                }
                num += __shfl_xor_sync(0xffffffffu, num, 1);
                num += __shfl_xor_sync(0xffffffffu, num, 2);
                nq += __shfl_xor_sync(0xffffffffu, nq, 1);
                nq += __shfl_xor_sync(0xffffffffu, nq, 2);
                if (part == 0 && col_ok) {
                    const float den = fmaxf(fabsf(nq), Ge[t]) + 1e-6f;
                    out[(((long long)b * Tn + t0 + t) * H + hd) * Dv + vc] = num / den;
                }
            }
        }
        // padding rows of the step: defined output
        for (int t = max(nt, 0); t < SC_TOK && t0 + t < Tn; ++t)
            if (part == 0 && col_ok) out[(((long long)b * Tn + t0 + t) * H + hd) * Dv + vc] = 0.f;
    }
    if (nb > 0) {
#pragma unroll
        for (int r = 0; r < DPT; ++r) {
            const int d = r * 4 + part;
            if (d < D) {
                if (col_ok) Sg[(long long)d * Dv + vc] = S[r];
                // n and m are read by every column slice of this (row, head): the new values go to a scratch row and
                // reach the state in a second launch, when no slice can still want the old ones
                if (blockIdx.x == 0 && col == 0) next_n[((long long)b * H + hd) * D + d] = nn[r];
            }
        }
        if (blockIdx.x == 0 && tid == 0) next_m[(long long)b * H + hd] = m_run;
    }
}

// One token per row (token generation): nothing is carried in registers between tokens, so the mapping is chosen for the
// state traffic alone -- a lane owns a value column (a warp reads 128 contiguous bytes of a state row), the four warps
// take every fourth row, partial sums meet in shared memory.  Any key size.
template <typename T>
__global__ void __launch_bounds__(128)
mlstm_step_kernel(const T* __restrict__ proj, long long ld, int q_off, int k_off, int v_off, const float* __restrict__ gi,
                  const float* __restrict__ gf, float* __restrict__ state_s, const float* __restrict__ state_n,
                  const float* __restrict__ state_m, float* __restrict__ next_n, float* __restrict__ next_m,
                  float* __restrict__ out, const int* __restrict__ q_start, const int* __restrict__ seq_ids, int H, int D,
                  int Dv, float qscale) {
    extern __shared__ float smem[];
    float* qs = smem;                         // [D]
    float* ks = qs + D;                       // [D]
    __shared__ float red[4][32];
    __shared__ float rednq[4];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int col = blockIdx.x * 32 + lane, hd = blockIdx.y, b = blockIdx.z;
    const bool col_ok = col < Dv;
    const int line = seq_ids != nullptr ? seq_ids[b] : b;
    const bool fresh = q_start[b] == 0;
    const T* row = proj + (long long)b * ld;
    for (int d = tid; d < D; d += 128) {
        qs[d] = ldf(row + q_off + hd * D + d) * qscale;
        ks[d] = ldf(row + k_off + hd * D + d);
    }
    const float f = gf[(long long)b * H + hd], i = gi[(long long)b * H + hd];
    const float m0 = fresh ? 0.f : state_m[(long long)line * H + hd];
    const float mn = fmaxf(f + m0, i);
    const float a = expf(f + m0 - mn), bw = expf(i - mn), e = expf(-mn);
    __syncthreads();
    const float vt = col_ok ? ldf(row + v_off + hd * Dv + col) * bw : 0.f;
    float* Sg = state_s + ((long long)line * H + hd) * D * Dv + col;
    float num = 0.f;
#pragma unroll 8
    for (int d = warp; d < D; d += 4) {
        const float s_old = (fresh || !col_ok) ? 0.f : Sg[(long long)d * Dv];
        const float sv = fmaf(a, s_old, ks[d] * vt);
        if (col_ok) Sg[(long long)d * Dv] = sv;
        num = fmaf(sv, qs[d], num);
    }
    const float* Ng = state_n + ((long long)line * H + hd) * D;
    float nq = 0.f;
    for (int d = tid; d < D; d += 128) {
        const float nv = fmaf(a, fresh ? 0.f : Ng[d], bw * ks[d]);
        nq = fmaf(nv, qs[d], nq);
        if (blockIdx.x == 0) next_n[((long long)b * H + hd) * D + d] = nv;
    }
    nq = warp_sum(nq);
    red[warp][lane] = num;
    if (lane == 0) rednq[warp] = nq;
    __syncthreads();
    if (warp == 0 && col_ok) {
        const float nsum = red[0][lane] + red[1][lane] + red[2][lane] + red[3][lane];
        const float nqt = rednq[0] + rednq[1] + rednq[2] + rednq[3];
        out[((long long)b * H + hd) * Dv + col] = nsum / (fmaxf(fabsf(nqt), e) + 1e-6f);
    }
    if (blockIdx.x == 0 && tid == 0) next_m[(long long)b * H + hd] = mn;
}

__global__ void mlstm_commit_kernel(const float* __restrict__ next_n, const float* __restrict__ next_m,
                                    float* __restrict__ state_n, float* __restrict__ state_m,
                                    const int* __restrict__ n_new, const int* __restrict__ seq_ids, int H, int D) {
    const int hd = blockIdx.x, b = blockIdx.y;
    if (n_new != nullptr && n_new[b] <= 0) return;
    const int line = seq_ids != nullptr ? seq_ids[b] : b;
    for (int d = threadIdx.x; d < D; d += blockDim.x)
        state_n[((long long)line * H + hd) * D + d] = next_n[((long long)b * H + hd) * D + d];
    if (threadIdx.x == 0) state_m[(long long)line * H + hd] = next_m[(long long)b * H + hd];
}

// Chunk-wise form of the same recurrence, the part that is sequential over chunks.  For chunk c of a (row, head) pair,
// u[c] holds the chunk's own contribution sum_s w_s k_s v_s^T (or sum_s w_s k_s), weighted relative to the chunk's local
// maximum mloc[c], and ftot[c] the sum of the chunk's log forget gates.  Walking the chunks in order,
//   m' = max(ftot[c] + m, mloc[c]);   s' = exp(ftot[c] + m - m') s + exp(mloc[c] - m') u[c]
// and u[c] is REPLACED by the state at the chunk's start (what the chunk's outputs need).  One thread per state element.
__global__ void mlstm_chunk_states_kernel(float* __restrict__ u, const float* __restrict__ ftot,
                                          const float* __restrict__ mloc, const float* __restrict__ s0,
                                          const float* __restrict__ m0, float* __restrict__ s_out,
                                          float* __restrict__ m_start, float* __restrict__ m_out, int NC, long long E) {
    const long long bh = blockIdx.y;
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E) return;
    float s = s0[bh * E + e];
    float m = m0[bh];
    constexpr int AHEAD = 8;                  // loads of the next chunks are issued before the stores of these
    for (int c0 = 0; c0 < NC; c0 += AHEAD) {
        float uv[AHEAD];
#pragma unroll
        for (int j = 0; j < AHEAD; ++j) uv[j] = c0 + j < NC ? u[(bh * NC + c0 + j) * E + e] : 0.f;
#pragma unroll
        for (int j = 0; j < AHEAD; ++j) {
            const int c = c0 + j;
            if (c < NC) {
                const float ft = ftot[bh * NC + c], ml = mloc[bh * NC + c];
                const float mn = fmaxf(ft + m, ml);
                const float a = expf(ft + m - mn), b = expf(ml - mn);
                u[(bh * NC + c) * E + e] = s;
                if (e == 0 && m_start != nullptr) m_start[bh * NC + c] = m;
                s = fmaf(a, s, b * uv[j]);
                m = mn;
            }
        }
    }
    s_out[bh * E + e] = s;
    if (e == 0 && m_out != nullptr) m_out[bh] = m;
}

template <typename T, int DPT>
int launch_scan(const void* proj, long long ld, int q_off, int k_off, int v_off, const float* gi, const float* gf,
                float* ss, float* sn, float* sm, float* nxn, float* nxm, float* out, const int* q_start, const int* n_new,
                const int* seq_ids, int B, int Tn, int H, int D, int Dv, float qscale, cudaStream_t st) {
    const size_t smem = (size_t)(SC_TOK * (2 * D + SC_COLS) + 3 * SC_TOK + 1) * sizeof(float);
    auto kern = mlstm_scan_kernel<T, DPT>;
    if (smem > 48 * 1024) NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((Dv + SC_COLS - 1) / SC_COLS, H, B);
    kern<<<grid, SC_THREADS, smem, st>>>((const T*)proj, ld, q_off, k_off, v_off, gi, gf, ss, sn, sm, nxn, nxm, out, q_start,
                                         n_new, seq_ids, Tn, H, D, Dv, qscale);
    NXD_LAUNCH_CHECK();
    mlstm_commit_kernel<<<dim3(H, B), 64, 0, st>>>(nxn, nxm, sn, sm, n_new, seq_ids, H, D);
    NXD_LAUNCH_CHECK();
    return 0;
}

template <typename T>
int dispatch_scan(const void* proj, long long ld, int q_off, int k_off, int v_off, const float* gi, const float* gf,
                  float* ss, float* sn, float* sm, float* nxn, float* nxm, float* out, const int* q_start,
                  const int* n_new, const int* seq_ids, int B, int Tn, int H, int D, int Dv, float qscale,
                  cudaStream_t st) {
    if (Tn == 1 && n_new == nullptr) {                 // token generation
        dim3 grid((Dv + 31) / 32, H, B);
        mlstm_step_kernel<T><<<grid, 128, (size_t)2 * D * sizeof(float), st>>>(
            (const T*)proj, ld, q_off, k_off, v_off, gi, gf, ss, sn, sm, nxn, nxm, out, q_start, seq_ids, H, D, Dv, qscale);
        NXD_LAUNCH_CHECK();
        mlstm_commit_kernel<<<dim3(H, B), 64, 0, st>>>(nxn, nxm, sn, sm, nullptr, seq_ids, H, D);
        NXD_LAUNCH_CHECK();
        return 0;
    }
#define NXD_SCAN_CASE(DPT)                                                                                             \
    if (D <= 4 * DPT)                                                                                                  \
        return launch_scan<T, DPT>(proj, ld, q_off, k_off, v_off, gi, gf, ss, sn, sm, nxn, nxm, out, q_start, n_new,   \
                                   seq_ids, B, Tn, H, D, Dv, qscale, st)
    NXD_SCAN_CASE(4);
    NXD_SCAN_CASE(8);
    NXD_SCAN_CASE(16);
    NXD_SCAN_CASE(32);
    NXD_SCAN_CASE(64);
    NXD_SCAN_CASE(96);
#undef NXD_SCAN_CASE
    NXD_REQUIRE(false, "recurrent mixer: key size %d above %d", D, 4 * 96);
    return 1;
}

// o [N, H, Dv] (TO) -> out [N, H * Dv] (T); gate [N, ld_g] (T) read at column g_off + c; weight [H * Dv] fp32 or NULL
template <typename TO, typename T>
__global__ void head_norm_gate_kernel(const TO* __restrict__ o, const T* __restrict__ gate, long long ld_g, int g_off,
                                      const float* __restrict__ weight, T* __restrict__ out, long long units, int H,
                                      int Dv, int normalize, float eps, int gate_act) {
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= units) return;
    const long long n = unit / H;
    const int hd = (int)(unit % H);
    const TO* src = o + unit * Dv;
    float r = 1.f;
    if (normalize) {
        float ss = 0.f;
        for (int c = lane; c < Dv; c += 32) {
            const float v = ldf(src + c);
            ss += v * v;
        }
        ss = warp_sum(ss);
        r = 1.f / sqrtf(ss / (float)Dv + eps);
    }
    const T* g = gate + n * ld_g + g_off + (long long)hd * Dv;
    T* dst = out + unit * Dv;
    for (int c = lane; c < Dv; c += 32) {
        float v = ldf(src + c) * r;
        if (weight != nullptr) v *= weight[hd * Dv + c];
        const float z = ldf(g + c);
        v *= (gate_act == 1 ? z : 1.f) / (1.f + expf(-z));      // 0: sigmoid(z), 1: silu(z) = z * sigmoid(z)
        stf(dst + c, v);
    }
}

template <typename T>
__global__ void relu_squared_kernel(const T* __restrict__ x, T* __restrict__ y, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float v = fmaxf(ldf(x + i), 0.f);
        stf(y + i, v * v);
    }
}

// bf16, 8 values (16 bytes) per thread; n8 = n / 8 full vectors, the tail goes through the scalar kernel
__global__ void relu_squared_vec_kernel(const bf16x8* __restrict__ x, bf16x8* __restrict__ y, long long n8) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n8) {
        float f[8];
        unpack8(x[i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float v = fmaxf(f[j], 0.f);
            f[j] = v * v;
        }
        y[i] = pack8(f);
    }
}

}  // namespace

// dtype (mixer input and gate rows): 0 = bf16, 1 = fp32
NXD_API int nxd_mlstm_gates(int dtype, const void* h, const void* w, const float* bias, float* gi, float* gf,
                            long long N, int W, int H, float cap, void* stream) {
    const long long units = N;
    if (units == 0 || H == 0) return 0;
    const int wpb = 8;
    const unsigned blocks = (unsigned)((units + wpb - 1) / wpb);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == 0)
        mlstm_gates_kernel<bf16><<<blocks, wpb * 32, 0, st>>>((const bf16*)h, (const bf16*)w, bias, gi, gf, units, W, H, cap);
    else
        mlstm_gates_kernel<float><<<blocks, wpb * 32, 0, st>>>((const float*)h, (const float*)w, bias, gi, gf, units, W, H,
                                                               cap);
    NXD_LAUNCH_CHECK();
    return 0;
}

// proj [B * Tn, ld]: queries, keys and values of the step at column offsets q_off / k_off / v_off (head-major);
// gi / gf [B * Tn, H] fp32 log-space gates; state of cache line seq_ids[b] (or b) is read (unless q_start[b] == 0) and
// written; next_n [B, H, D] and next_m [B, H]: scratch; out [B * Tn, H, Dv] fp32.
NXD_API int nxd_mlstm_scan(int dtype, const void* proj, long long ld, int q_off, int k_off, int v_off, const float* gi,
                           const float* gf, float* state_s, float* state_n, float* state_m, float* next_n,
                           float* next_m, float* out,
                           const int* q_start, const int* n_new, const int* seq_ids, int B, int Tn, int H, int D, int Dv,
                           float qscale, void* stream) {
    if (B * Tn == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == 0)
        return dispatch_scan<bf16>(proj, ld, q_off, k_off, v_off, gi, gf, state_s, state_n, state_m, next_n, next_m, out,
                                   q_start, n_new, seq_ids, B, Tn, H, D, Dv, qscale, st);
    return dispatch_scan<float>(proj, ld, q_off, k_off, v_off, gi, gf, state_s, state_n, state_m, next_n, next_m, out,
                                q_start, n_new, seq_ids, B, Tn, H, D, Dv, qscale, st);
}

// o_dtype: dtype of o (0 bf16, 1 fp32); dtype: gate and output
NXD_API int nxd_head_norm_gate(int o_dtype, int dtype, const void* o, const void* gate, long long ld_g, int g_off,
                               const float* weight, void* out, long long N, int H, int Dv, int normalize, float eps,
                               int gate_act, void* stream) {
    const long long units = N * H;
    if (units == 0) return 0;
    const int wpb = 8;
    const unsigned blocks = (unsigned)((units + wpb - 1) / wpb);
    cudaStream_t st = (cudaStream_t)stream;
    if (o_dtype == 1 && dtype == 0)
        head_norm_gate_kernel<float, bf16><<<blocks, wpb * 32, 0, st>>>((const float*)o, (const bf16*)gate, ld_g, g_off,
                                                                        weight, (bf16*)out, units, H, Dv, normalize, eps,
                                                                        gate_act);
    else if (o_dtype == 1 && dtype == 1)
        head_norm_gate_kernel<float, float><<<blocks, wpb * 32, 0, st>>>((const float*)o, (const float*)gate, ld_g, g_off,
                                                                         weight, (float*)out, units, H, Dv, normalize, eps,
                                                                         gate_act);
    else if (o_dtype == 0 && dtype == 0)
        head_norm_gate_kernel<bf16, bf16><<<blocks, wpb * 32, 0, st>>>((const bf16*)o, (const bf16*)gate, ld_g, g_off,
                                                                       weight, (bf16*)out, units, H, Dv, normalize, eps,
                                                                       gate_act);
    else
        NXD_REQUIRE(false, "head norm / gate: dtypes %d -> %d", o_dtype, dtype);
    NXD_LAUNCH_CHECK();
    return 0;
}

NXD_API int nxd_relu_squared(int dtype, const void* x, void* y, long long n, void* stream) {
    if (n == 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0 && n >= 8) {
        const long long n8 = n / 8;
        relu_squared_vec_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const bf16x8*)x, (bf16x8*)y,
                                                                                               n8);
        NXD_LAUNCH_CHECK();
        if (n8 * 8 == n) return 0;
        const long long rest = n - n8 * 8;
        relu_squared_kernel<bf16><<<1, 256, 0, (cudaStream_t)stream>>>((const bf16*)x + n8 * 8, (bf16*)y + n8 * 8, rest);
    } else if (dtype == 0)
        relu_squared_kernel<bf16><<<blocks, 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y, n);
    else
        relu_squared_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((const float*)x, (float*)y, n);
    NXD_LAUNCH_CHECK();
    return 0;
}

// u [BH, NC, E] fp32 (in: per-chunk contributions, out: state at every chunk's start); ftot, mloc [BH, NC]; s0 [BH, E],
// m0 [BH]: state before the first chunk; s_out [BH, E]: state after the last; m_start [BH, NC] and m_out [BH] may be NULL.
NXD_API int nxd_mlstm_chunk_states(float* u, const float* ftot, const float* mloc, const float* s0, const float* m0,
                                   float* s_out, float* m_start, float* m_out, long long BH, int NC, long long E,
                                   void* stream) {
    if (BH == 0 || E == 0) return 0;
    NXD_REQUIRE(BH < 65536, "recurrent mixer: %lld (row, head) pairs in one launch", BH);
    dim3 grid((unsigned)((E + 255) / 256), (unsigned)BH);
    mlstm_chunk_states_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(u, ftot, mloc, s0, m0, s_out, m_start, m_out, NC, E);
    NXD_LAUNCH_CHECK();
    return 0;
}
