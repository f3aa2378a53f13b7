// Retention: linear attention with a fixed decay per head and no softmax or denominator, over a per-sequence state that
// lives in fp32 device memory.
//
//   S_t = decay_h S_{t-1} + k_t v_t^T          S: [D, Dv] per head
//   o_t = S_t^T q_t
//
// Queries and keys come as bf16 / fp32 projection columns; they are rotated here (optional: the first `rot` dimensions
// of every head turn by the angle of (position, pair), pairs (i, i + rot / 2) or (2i, 2i + 1), cos / sin from tables
// [positions, rot / 2]) and the keys are multiplied by kscale after the rotation.  Rotation, products, decay and state
// are fp32; this file is compiled without fast-math.
//
// Kernels:
//   retention_scan     one CTA per (value-column slice, head, batch row): the slice S[:, v0 : v0 + 32] stays in
//                      registers (4 lanes per column, each holding every 4th row), the step's tokens stream through
//                      shared memory in blocks of 16.  A row that starts at position 0 starts from the zero state, any
//                      other row continues from the state of its line; padding tokens (t >= n_new[b]) change nothing.
//                      Serves token generation (one token), short steps and fp32 serving.
//   retention_chunk_*  the chunk-wise form for long steps, three kernels (4 x 4 register tiles, value columns in tiles):
//                        local   per (chunk, head, row, column tile): rotated q / k of the chunk in shared memory,
//                                P[t][s] = decay^(t-s) (q_t . k_s) for s <= t, o_local = P v, and the chunk's own
//                                contribution to the state U = sum_s decay^(L-1-s) k_s v_s^T
//                        states  per (head, row), sequential over chunks: state at every chunk's start (in place of U),
//                                and the line's state after the step
//                        cross   o_t += decay^(t+1) S_c^T q_t
#include "common.cuh"

namespace {

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }

// element d of a head's rotated row; x points at the head's first column
template <typename T>
__device__ __forceinline__ float rotated(const T* x, int d, int rot, int halves, const float* cs, const float* sn) {
    const float a = ldf(x + d);
    if (d >= rot) return a;
    int i, partner;
    bool first;
    if (halves) {
        first = d < rot / 2;
        i = first ? d : d - rot / 2;
        partner = first ? d + rot / 2 : d - rot / 2;
    } else {
        first = (d & 1) == 0;
        i = d >> 1;
        partner = first ? d + 1 : d - 1;
    }
    const float b = ldf(x + partner);
    return first ? a * cs[i] - b * sn[i] : a * cs[i] + b * sn[i];
}

constexpr int SC_THREADS = 128, SC_COLS = 32, SC_TOK = 16;

// proj [B * Tn, ld]: head hd of q at column q_off + hd * D, of k at k_off + hd * D, of v at v_off + hd * Dv.
// state [lines, H, D, Dv] fp32; out [B * Tn, H, Dv] fp32.
template <typename T, int DPT>
__global__ void __launch_bounds__(SC_THREADS)
retention_scan_kernel(const T* __restrict__ proj, long long ld, int q_off, int k_off, int v_off,
                      const float* __restrict__ decay, float* __restrict__ state, float* __restrict__ out,
                      const int* __restrict__ q_start, const int* __restrict__ n_new, const int* __restrict__ seq_ids,
                      int Tn, int H, int D, int Dv, float kscale, const float* __restrict__ rope_cos,
                      const float* __restrict__ rope_sin, int rot, int halves, int max_pos) {
    extern __shared__ float smem[];
    float* Qs = smem;                         // [SC_TOK][D]
    float* Ks = Qs + SC_TOK * D;              // [SC_TOK][D]
    float* Vs = Ks + SC_TOK * D;              // [SC_TOK][SC_COLS]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int col = warp * 8 + (lane >> 2), part = lane & 3;      // 4 lanes share a value column
    const int v0 = blockIdx.x * SC_COLS, hd = blockIdx.y, b = blockIdx.z;
    const int vc = v0 + col;
    const bool col_ok = vc < Dv;
    const int nb = n_new != nullptr ? min(n_new[b], Tn) : Tn;
    const int line = seq_ids != nullptr ? seq_ids[b] : b;
    const int p0 = q_start[b];
    const bool fresh = p0 == 0;
    const float a = decay[hd];
    float* Sg = state + ((long long)line * H + hd) * D * Dv;

    float S[DPT];
#pragma unroll
    for (int r = 0; r < DPT; ++r) {
        const int d = r * 4 + part;
        S[r] = (d < D && !fresh && col_ok) ? Sg[(long long)d * Dv + vc] : 0.f;
    }

    for (int t0 = 0; t0 < Tn; t0 += SC_TOK) {
        const int nt = min(SC_TOK, nb - t0);          // real tokens of this block (may be <= 0: only padding left)
        __syncthreads();
        if (nt > 0) {
            for (int idx = tid; idx < nt * D; idx += SC_THREADS) {
                const int t = idx / D, d = idx - t * D;
                const T* row = proj + ((long long)b * Tn + t0 + t) * ld;
                int pos = p0 + t0 + t;
                pos = pos < max_pos ? pos : max_pos - 1;
                const float* cs = rope_cos != nullptr ? rope_cos + (long long)pos * (rot / 2) : nullptr;
                const float* sn = rope_cos != nullptr ? rope_sin + (long long)pos * (rot / 2) : nullptr;
                const int r = rope_cos != nullptr ? rot : 0;
                Qs[idx] = rotated(row + q_off + hd * D, d, r, halves, cs, sn);
                Ks[idx] = rotated(row + k_off + hd * D, d, r, halves, cs, sn) * kscale;
            }
            for (int idx = tid; idx < nt * SC_COLS; idx += SC_THREADS) {
                const int t = idx / SC_COLS, c = idx - t * SC_COLS;
                const T* row = proj + ((long long)b * Tn + t0 + t) * ld;
                Vs[idx] = (v0 + c < Dv) ? ldf(row + v_off + hd * Dv + v0 + c) : 0.f;
            }
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float vt = Vs[t * SC_COLS + col];
            const float* qr = Qs + t * D;
            const float* kr = Ks + t * D;
            float num = 0.f;
#pragma unroll
            for (int r = 0; r < DPT; ++r) {
                const int d = r * 4 + part;
                if (d < D) {
                    S[r] = fmaf(a, S[r], kr[d] * vt);
                    num = fmaf(S[r], qr[d], num);
                }
            }
            num += __shfl_xor_sync(0xffffffffu, num, 1);
            num += __shfl_xor_sync(0xffffffffu, num, 2);
            if (part == 0 && col_ok) out[(((long long)b * Tn + t0 + t) * H + hd) * Dv + vc] = num;
        }
        // padding rows of the step: defined output
        for (int t = max(nt, 0); t < SC_TOK && t0 + t < Tn; ++t)
            if (part == 0 && col_ok) out[(((long long)b * Tn + t0 + t) * H + hd) * Dv + vc] = 0.f;
    }
    if (nb > 0 && col_ok) {
#pragma unroll
        for (int r = 0; r < DPT; ++r) {
            const int d = r * 4 + part;
            if (d < D) Sg[(long long)d * Dv + vc] = S[r];
        }
    }
}

template <typename T>
int dispatch_scan(const void* proj, long long ld, int q_off, int k_off, int v_off, const float* decay, float* state,
                  float* out, const int* q_start, const int* n_new, const int* seq_ids, int B, int Tn, int H, int D, int Dv,
                  float kscale, const float* rope_cos, const float* rope_sin, int rot, int halves, int max_pos,
                  cudaStream_t st) {
    dim3 grid((Dv + SC_COLS - 1) / SC_COLS, H, B);
    const size_t smem = (size_t)(2 * SC_TOK * D + SC_TOK * SC_COLS) * sizeof(float);
#define NXD_RT_SCAN(DPT)                                                                                              \
    do {                                                                                                              \
        auto kern = retention_scan_kernel<T, DPT>;                                                                    \
        if (smem > 48 * 1024)                                                                                         \
            NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));       \
        kern<<<grid, SC_THREADS, smem, st>>>((const T*)proj, ld, q_off, k_off, v_off, decay, state, out, q_start, n_new, \
                                             seq_ids, Tn, H, D, Dv, kscale, rope_cos, rope_sin, rot, halves, max_pos); \
    } while (0)
    if (D <= 32) NXD_RT_SCAN(8);
    else if (D <= 64) NXD_RT_SCAN(16);
    else if (D <= 128) NXD_RT_SCAN(32);
    else if (D <= 256) NXD_RT_SCAN(64);
    else NXD_REQUIRE(false, "retention: key size %d above 256", D);
#undef NXD_RT_SCAN
    NXD_LAUNCH_CHECK();
    return 0;
}

// ---- chunk-wise form -------------------------------------------------------------------------------------------------
// The products are register-tiled: a thread owns a 4 x 4 tile of outputs, reads four scalars of one operand and a
// float4 of the other per step, so a step of 16 multiply-adds costs five shared-memory loads.  The value columns are
// walked in tiles of at most 128 inside the CTA, so that any head size fits in shared memory.
constexpr int CH = 64, CH_THREADS = 256, VT_MAX = 128, PP = CH + 1;

__device__ __forceinline__ void fma44(float (&acc)[4][4], const float (&a)[4], const float4 b) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        acc[i][0] = fmaf(a[i], b.x, acc[i][0]);
        acc[i][1] = fmaf(a[i], b.y, acc[i][1]);
        acc[i][2] = fmaf(a[i], b.z, acc[i][2]);
        acc[i][3] = fmaf(a[i], b.w, acc[i][3]);
    }
}

// stages the chunk's queries and keys: raw projection columns into shared memory (independent loads), then the rotation
// of the pairs in place; the keys carry kscale (a scale commutes with the rotation)
template <typename T>
__device__ __forceinline__ void stage_qk(const T* __restrict__ proj, long long ld, int q_off, int k_off, long long row0,
                                         int hd, int D, int DP, int nt, int p0, float kscale, float* Qs, float* Ks,
                                         const float* __restrict__ rope_cos, const float* __restrict__ rope_sin, int rot,
                                         int halves, int max_pos, bool want_k) {
    const int tid = threadIdx.x;
#pragma unroll 8
    for (int idx = tid; idx < CH * D; idx += CH_THREADS) {
        const int t = idx / D, d = idx - t * D;
        const T* row = proj + (row0 + t) * ld + hd * D + d;
        Qs[t * DP + d] = t < nt ? ldf(row + q_off) : 0.f;
        if (want_k) Ks[t * DP + d] = t < nt ? ldf(row + k_off) * kscale : 0.f;
    }
    if (rope_cos == nullptr || rot <= 0) return;
    __syncthreads();
    const int half = rot / 2;
#pragma unroll 4
    for (int idx = tid; idx < nt * half; idx += CH_THREADS) {
        const int t = idx / half, i = idx - t * half;
        const int iu = halves ? i : 2 * i, iv = halves ? i + half : 2 * i + 1;
        int pos = p0 + t;
        pos = pos < max_pos ? pos : max_pos - 1;
        const float c = rope_cos[(long long)pos * half + i], sn = rope_sin[(long long)pos * half + i];
        float u = Qs[t * DP + iu], v = Qs[t * DP + iv];
        Qs[t * DP + iu] = u * c - v * sn;
        Qs[t * DP + iv] = v * c + u * sn;
        if (want_k) {
            u = Ks[t * DP + iu], v = Ks[t * DP + iv];
            Ks[t * DP + iu] = u * c - v * sn;
            Ks[t * DP + iv] = v * c + u * sn;
        }
    }
}

// grid (chunks, H, B).  Shared: Vs [CH][VT], P [CH][CH + 1], Qs [CH][D + 1], Ks [CH][D + 1]; the value columns are
// walked in tiles of VT.  out [B * Tn, H, Dv] gets the chunk-local part; U [B, H, NC, D, Dv] the chunk's contribution to
// the state; qrot [B * Tn, H, D] keeps the rotated queries for the cross-chunk pass.
template <typename T>
__global__ void __launch_bounds__(CH_THREADS)
retention_chunk_local_kernel(const T* __restrict__ proj, long long ld, int q_off, int k_off, int v_off,
                             const float* __restrict__ decay, float* __restrict__ out, float* __restrict__ U,
                             float* __restrict__ qrot, const int* __restrict__ q_start, const int* __restrict__ n_new,
                             int Tn, int NC, int H, int D, int Dv, int VT, int NVT, float kscale,
                             const float* __restrict__ rope_cos, const float* __restrict__ rope_sin, int rot, int halves,
                             int max_pos) {
    extern __shared__ __align__(16) float smem[];
    const int DP = D + 1;
    float* Vs = smem;                          // [CH][VT], 16-byte aligned rows
    float* P = Vs + CH * VT;                   // [CH][PP]
    float* Qs = P + CH * PP;                   // [CH][DP]
    float* Ks = Qs + CH * DP;                  // [CH][DP]
    __shared__ float pw[CH + 1];               // decay^j
    const int c = blockIdx.x, hd = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
    const int nb = n_new != nullptr ? min(n_new[b], Tn) : Tn;
    const int t0 = c * CH;
    const int nt = max(0, min(CH, nb - t0));   // real tokens of this chunk
    const float a = decay[hd];
    if (tid <= CH) pw[tid] = powf(a, (float)tid);
    stage_qk(proj, ld, q_off, k_off, (long long)b * Tn + t0, hd, D, DP, nt, q_start[b] + t0, kscale, Qs, Ks, rope_cos,
             rope_sin, rot, halves, max_pos, true);
    __syncthreads();
    for (int idx = tid; idx < nt * D; idx += CH_THREADS) {
        const int t = idx / D, d = idx - t * D;
        qrot[(((long long)b * Tn + t0 + t) * H + hd) * D + d] = Qs[t * DP + d];
    }
    // P[t][s] = decay^(t - s) (q_t . k_s), s <= t: one 4 x 4 tile per thread, tiles above the diagonal are zero
    {
        const int tg = tid >> 4, sg = tid & 15;
        float acc[4][4] = {};
        if (sg <= tg && 4 * tg < nt) {
            const float* qr = Qs + 4 * tg * DP;
            const float* kr = Ks + 4 * sg * DP;
#pragma unroll 4
            for (int d = 0; d < D; ++d) {
                const float qa[4] = {qr[d], qr[DP + d], qr[2 * DP + d], qr[3 * DP + d]};
                fma44(acc, qa, make_float4(kr[d], kr[DP + d], kr[2 * DP + d], kr[3 * DP + d]));
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int t = 4 * tg + i, sx = 4 * sg + j;
                P[t * PP + sx] = (sx <= t && t < nt) ? acc[i][j] * pw[t - sx] : 0.f;
            }
    }
    const int JG = VT / 4;
    const bool vec_out = (Dv & 3) == 0;
    float* Ug = U + (((long long)b * H + hd) * NC + c) * D * Dv;
    const int DG = (D + 3) / 4;
    for (int v0 = 0; v0 < Dv; v0 += VT) {
        __syncthreads();                       // P is complete; the previous tile's readers of Vs are done
#pragma unroll 8
        for (int idx = tid; idx < CH * VT; idx += CH_THREADS) {
            const int t = idx / VT, j = idx - t * VT;
            Vs[idx] = (t < nt && v0 + j < Dv) ? ldf(proj + ((long long)b * Tn + t0 + t) * ld + v_off + hd * Dv + v0 + j) : 0.f;
        }
        __syncthreads();
        // o_local[t][j] = sum_{s <= t} P[t][s] v[s][j]
        for (int tile = tid; tile < (CH / 4) * JG; tile += CH_THREADS) {
            const int tg = tile / JG, jg = tile - tg * JG;
            float acc[4][4] = {};
            const int s_end = min(4 * tg + 4, nt);
            const float* pr = P + 4 * tg * PP;
#pragma unroll 4
            for (int sx = 0; sx < s_end; ++sx) {
                const float pa[4] = {pr[sx], pr[PP + sx], pr[2 * PP + sx], pr[3 * PP + sx]};
                fma44(acc, pa, *reinterpret_cast<const float4*>(Vs + sx * VT + 4 * jg));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int t = 4 * tg + i, j = v0 + 4 * jg;
                if (t0 + t >= Tn || j >= Dv) continue;
                float* dst = out + (((long long)b * Tn + t0 + t) * H + hd) * Dv + j;
                if (vec_out) {
                    *reinterpret_cast<float4*>(dst) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
                } else {
#pragma unroll
                    for (int x = 0; x < 4; ++x)
                        if (j + x < Dv) dst[x] = acc[i][x];
                }
            }
        }
        // U[d][j] = sum_s decay^(nt - 1 - s) k_s[d] v_s[j]: the state the chunk's real tokens add, seen from its end
        for (int tile = tid; tile < DG * JG; tile += CH_THREADS) {
            const int dg = tile / JG, jg = tile - dg * JG;
            float acc[4][4] = {};
#pragma unroll 4
            for (int sx = 0; sx < nt; ++sx) {
                const float w = pw[nt - 1 - sx];
                const float* kr = Ks + sx * DP + 4 * dg;
                float ka[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) ka[i] = (4 * dg + i < D) ? kr[i] * w : 0.f;
                fma44(acc, ka, *reinterpret_cast<const float4*>(Vs + sx * VT + 4 * jg));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int d = 4 * dg + i, j = v0 + 4 * jg;
                if (d >= D || j >= Dv) continue;
                float* dst = Ug + (long long)d * Dv + j;
                if (vec_out) {
                    *reinterpret_cast<float4*>(dst) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
                } else {
#pragma unroll
                    for (int x = 0; x < 4; ++x)
                        if (j + x < Dv) dst[x] = acc[i][x];
                }
            }
        }
    }
}

// grid (ceil(D * Dv / 256), H, B): every thread walks the chunks of one state element, eight chunks' loads in flight at a
// time: U[c] <- state at the start of chunk c; the line's state <- state after the step.
__global__ void retention_chunk_states_kernel(float* __restrict__ U, float* __restrict__ state,
                                              const float* __restrict__ decay, const int* __restrict__ q_start,
                                              const int* __restrict__ n_new, const int* __restrict__ seq_ids, int Tn,
                                              int NC, int H, long long E) {
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E) return;
    const int hd = blockIdx.y, b = blockIdx.z;
    const int nb = n_new != nullptr ? min(n_new[b], Tn) : Tn;
    const int line = seq_ids != nullptr ? seq_ids[b] : b;
    float* Sg = state + ((long long)line * H + hd) * E + e;
    float s = q_start[b] == 0 ? 0.f : *Sg;
    const float a = decay[hd];
    const float full = powf(a, (float)CH);
    float* u = U + ((long long)b * H + hd) * NC * E + e;
    for (int c0 = 0; c0 < NC; c0 += 8) {
        float uc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) uc[i] = c0 + i < NC ? u[(long long)(c0 + i) * E] : 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (c0 + i >= NC) break;
            const int nt = max(0, min(CH, nb - (c0 + i) * CH));
            u[(long long)(c0 + i) * E] = s;
            if (nt > 0) s = fmaf(nt == CH ? full : powf(a, (float)nt), s, uc[i]);
        }
    }
    if (nb > 0) *Sg = s;
}

// grid (chunks, H, B): out[t][j] += decay^(t + 1) sum_d S_c[d][j] q_t[d].  Shared: Ss [D][VT], Qs [CH][D]; the value
// columns are walked in tiles of VT.
__global__ void __launch_bounds__(CH_THREADS)
retention_chunk_cross_kernel(const float* __restrict__ U, const float* __restrict__ qrot, const float* __restrict__ decay,
                             float* __restrict__ out, const int* __restrict__ q_start, const int* __restrict__ n_new,
                             int Tn, int NC, int H, int D, int Dv, int VT, int NVT) {
    extern __shared__ __align__(16) float smem[];
    float* Ss = smem;                           // [D][VT]
    float* Qs = Ss + D * VT;                    // [CH][D]
    const int c = blockIdx.x, hd = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
    if (c == 0 && q_start[b] == 0) return;      // the first chunk of a fresh sequence starts from zero
    const int nb = n_new != nullptr ? min(n_new[b], Tn) : Tn;
    const int t0 = c * CH;
    const int nt = max(0, min(CH, nb - t0));
    if (nt == 0) return;
    const float a = decay[hd];
    const float* Sg = U + (((long long)b * H + hd) * NC + c) * D * Dv;
#pragma unroll 8
    for (int idx = tid; idx < CH * D; idx += CH_THREADS) {
        const int t = idx / D, d = idx - t * D;
        Qs[idx] = t < nt ? qrot[(((long long)b * Tn + t0 + t) * H + hd) * D + d] : 0.f;
    }
    const int JG = VT / 4;
    for (int v0 = 0; v0 < Dv; v0 += VT) {
        __syncthreads();
#pragma unroll 8
        for (int idx = tid; idx < D * VT; idx += CH_THREADS) {
            const int d = idx / VT, j = idx - d * VT;
            Ss[idx] = v0 + j < Dv ? Sg[(long long)d * Dv + v0 + j] : 0.f;
        }
        __syncthreads();
        for (int tile = tid; tile < (CH / 4) * JG; tile += CH_THREADS) {
            const int tg = tile / JG, jg = tile - tg * JG;
            if (4 * tg >= nt) continue;
            float acc[4][4] = {};
            const float* qr = Qs + 4 * tg * D;
#pragma unroll 4
            for (int d = 0; d < D; ++d) {
                const float qa[4] = {qr[d], qr[D + d], qr[2 * D + d], qr[3 * D + d]};
                fma44(acc, qa, *reinterpret_cast<const float4*>(Ss + d * VT + 4 * jg));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int t = 4 * tg + i, j = v0 + 4 * jg;
                if (t >= nt || j >= Dv) continue;
                const float w = powf(a, (float)(t + 1));
                float* dst = out + (((long long)b * Tn + t0 + t) * H + hd) * Dv + j;
#pragma unroll
                for (int x = 0; x < 4; ++x)
                    if (j + x < Dv) dst[x] = fmaf(w, acc[i][x], dst[x]);
            }
        }
    }
}

}  // namespace

// dtype of proj: 0 = bf16, 1 = fp32.  decay [H] fp32.  The state of cache line seq_ids[b] (or b) is read (unless
// q_start[b] == 0) and written.  rope_cos / rope_sin [max_pos, rot / 2] fp32 or NULL; halves: pairs (i, i + rot / 2).
NXD_API int nxd_retention_scan(int dtype, const void* proj, long long ld, int q_off, int k_off, int v_off,
                               const float* decay, float* state, float* out, const int* q_start, const int* n_new,
                               const int* seq_ids, int B, int Tn, int H, int D, int Dv, float kscale,
                               const float* rope_cos, const float* rope_sin, int rot, int halves, int max_pos,
                               void* stream) {
    if (B * Tn == 0) return 0;
    NXD_REQUIRE(rope_cos == nullptr || (rot % 2 == 0 && rot <= D && max_pos > 0), "retention: rotation over %d of %d", rot, D);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == 0)
        return dispatch_scan<bf16>(proj, ld, q_off, k_off, v_off, decay, state, out, q_start, n_new, seq_ids, B, Tn, H, D,
                                   Dv, kscale, rope_cos, rope_sin, rot, halves, max_pos, st);
    return dispatch_scan<float>(proj, ld, q_off, k_off, v_off, decay, state, out, q_start, n_new, seq_ids, B, Tn, H, D, Dv,
                                kscale, rope_cos, rope_sin, rot, halves, max_pos, st);
}

// The same step in chunks of 64 tokens.  U [B, H, ceil(Tn / 64), D, Dv] and qrot [B * Tn, H, D] are fp32 scratch.
NXD_API int nxd_retention_chunkwise(int dtype, const void* proj, long long ld, int q_off, int k_off, int v_off,
                                    const float* decay, float* state, float* out, float* U, float* qrot,
                                    const int* q_start, const int* n_new, const int* seq_ids, int B, int Tn, int H, int D,
                                    int Dv, float kscale, const float* rope_cos, const float* rope_sin, int rot,
                                    int halves, int max_pos, void* stream) {
    if (B * Tn == 0) return 0;
    NXD_REQUIRE(rope_cos == nullptr || (rot % 2 == 0 && rot <= D && max_pos > 0), "retention: rotation over %d of %d", rot, D);
    cudaStream_t st = (cudaStream_t)stream;
    const int NC = (Tn + CH - 1) / CH;
    const int VT = min(VT_MAX, (Dv + 3) / 4 * 4), NVT = (Dv + VT - 1) / VT;
    dim3 grid(NC, H, B);
    const size_t smem1 = (size_t)(2 * CH * (D + 1) + CH * PP + CH * VT) * sizeof(float);
    const size_t smem3 = (size_t)(D * VT + CH * D) * sizeof(float);
    NXD_REQUIRE(smem1 <= 220 * 1024 && smem3 <= 220 * 1024, "retention: key size %d too large for the chunk-wise form", D);
    NXD_REQUIRE(B < 65536, "retention: %d rows", B);
    if (dtype == 0) {
        auto kern = retention_chunk_local_kernel<bf16>;
        if (smem1 > 48 * 1024)
            NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1));
        kern<<<grid, CH_THREADS, smem1, st>>>((const bf16*)proj, ld, q_off, k_off, v_off, decay, out, U, qrot, q_start, n_new,
                                              Tn, NC, H, D, Dv, VT, NVT, kscale, rope_cos, rope_sin, rot, halves, max_pos);
    } else {
        auto kern = retention_chunk_local_kernel<float>;
        if (smem1 > 48 * 1024)
            NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1));
        kern<<<grid, CH_THREADS, smem1, st>>>((const float*)proj, ld, q_off, k_off, v_off, decay, out, U, qrot, q_start,
                                              n_new, Tn, NC, H, D, Dv, VT, NVT, kscale, rope_cos, rope_sin, rot, halves,
                                              max_pos);
    }
    NXD_LAUNCH_CHECK();
    const long long E = (long long)D * Dv;
    dim3 grid2((unsigned)((E + 255) / 256), H, B);
    retention_chunk_states_kernel<<<grid2, 256, 0, st>>>(U, state, decay, q_start, n_new, seq_ids, Tn, NC, H, E);
    NXD_LAUNCH_CHECK();
    if (smem3 > 48 * 1024)
        NXD_CHECK_CUDA(cudaFuncSetAttribute(retention_chunk_cross_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)smem3));
    retention_chunk_cross_kernel<<<grid, CH_THREADS, smem3, st>>>(U, qrot, decay, out, q_start, n_new, Tn, NC, H, D, Dv, VT,
                                                                  NVT);
    NXD_LAUNCH_CHECK();
    return 0;
}
