// Attention over the KV cache with a sliding window, kept first tokens ("sinks") and a linear distance bias, for
// per-head query/key size D and value size Dv that need not be equal or a power of two; bf16 or fp32 activations.
//
//   visible(i, j) = j <= i and (window <= 0 or i - j < window or j < keep_first)
//                   and (chunk <= 0 or floor(i / chunk) == floor(j / chunk))
//   score(i, j)   = scale * <q_i, k_j> - slope_h * (i - j)            (slopes == NULL: no bias)
//   softmax denominator = sum over visible j of exp(score) (+ exp(sink_h) with sinks != NULL: a learned per-head
//                   logit attached to no position that only takes probability mass)
// Chunk boundaries sit at absolute multiples of the chunk size.  The value rows may be a column range of the key rows (one
// cache tensor, value row pitch = key row pitch): the latent cache of a compressed key/value projection.
//
// Kernels:
//   window_attn_prefill_mma  bf16, head sizes from a compiled list: tensor-core prefill (see below); the generic prefill
//                         kernel serves every other case (fp32, other sizes)
//   qk_norm_cache_write   rows of the fused projection output -> unit-RMS q (written out) and unit-RMS k + v written
//                         into the cache at (line, position); statistics in fp32
//   window_attn_prefill   a tile of 16 queries of one head per CTA, keys and values streamed from the cache in tiles of
//                         32 rows, key tiles that no query of the tile can see are skipped, online softmax in fp32
//   window_attn_decode    one new token per row: one CTA per (row, key/value head), the warps split the visible keys
//                         (kept first tokens, then the window), every warp keeps an online-softmax state for the query
//                         heads of the group, merged through shared memory
// The cache is contiguous [lines, G, S, D] or paged [pages, G, page, D] with a block table [lines, cols].
#include "common.cuh"
#include "mma_sync.cuh"

namespace {

struct CacheAddr {
    long long stride_line, stride_head;   // elements
    const int* block_table;
    int page_size, table_cols, row_dim;
    int head_mod;                         // > 0: head g reads head g % head_mod (value heads shared by groups of key heads)
    __device__ __forceinline__ long long row(int line, int g, int pos) const {
        if (head_mod > 0) g %= head_mod;
        if (block_table != nullptr) {
            const int page = block_table[(long long)line * table_cols + pos / page_size];
            return (long long)page * stride_line + (long long)g * stride_head + (long long)(pos % page_size) * row_dim;
        }
        return (long long)line * stride_line + (long long)g * stride_head + (long long)pos * row_dim;
    }
};

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// ---------------------------------------------------------------------------------------------------------------------
// 1 / rms over all query heads (stat[2n]) and over all key heads (stat[2n + 1]) of projection row n: one warp per row
template <typename T>
__global__ void qk_row_stat_kernel(const T* __restrict__ qkv, long long ld, float* __restrict__ stat, long long rows, int nq,
                                   int nk, float eps) {
    const int lane = threadIdx.x & 31;
    const long long n = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= rows) return;
    const T* row = qkv + n * ld;
    float sq = 0.f, sk = 0.f;
    for (int i = lane; i < nq; i += 32) {
        const float v = ldf(row + i);
        sq += v * v;
    }
    for (int i = lane; i < nk; i += 32) {
        const float v = ldf(row + nq + i);
        sk += v * v;
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    if (lane == 0) {
        stat[2 * n] = 1.f / sqrtf(sq / (float)nq + eps);
        stat[2 * n + 1] = nk > 0 ? 1.f / sqrtf(sk / (float)nk + eps) : 1.f;
    }
}

template <typename T>
__global__ void qk_norm_cache_write_kernel(const T* __restrict__ qkv, long long ld, T* __restrict__ q_out,
                                           T* __restrict__ cache_k, T* __restrict__ cache_v, CacheAddr ka, CacheAddr va,
                                           const int* __restrict__ q_start, const int* __restrict__ n_new,
                                           const int* __restrict__ seq_ids, long long units, int Tn, int H, int G, int D,
                                           int Dv, int has_kv, int normalize, float eps, int max_pos, int writeback,
                                           const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                                           const float* __restrict__ rope_cos, const float* __restrict__ rope_sin,
                                           int rope_dims, int value_from_key, int Gv, int rope_halves,
                                           int whole_norm, const float* __restrict__ row_stat) {
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= units) return;
    const int per_row = H + (has_kv ? G + Gv : 0);
    const long long n = unit / per_row;
    const int hd = (int)(unit % per_row);
    const int b = (int)(n / Tn), t = (int)(n % Tn);
    const T* src;
    int dim;
    if (hd < H) {
        src = qkv + n * ld + (long long)hd * D;
        dim = D;
    } else if (hd < H + G) {
        src = qkv + n * ld + (long long)H * D + (long long)(hd - H) * D;
        dim = D;
    } else if (value_from_key) {             // the raw key projections double as values: no value columns in the row
        src = qkv + n * ld + (long long)H * D + (long long)(hd - H - G) * D;
        dim = Dv;
    } else {
        src = qkv + n * ld + (long long)(H + G) * D + (long long)(hd - H - G) * Dv;
        dim = Dv;
    }
    T* dst;
    if (hd < H) {
        dst = q_out + (n * H + hd) * D;
    } else {
        const bool valid = n_new == nullptr || t < n_new[b];
        const int pos = q_start[b] + t;
        if (!valid || pos >= max_pos || pos < 0) return;
        const int line = seq_ids != nullptr ? seq_ids[b] : b;
        dst = hd < H + G ? cache_k + ka.row(line, hd - H, pos) : cache_v + va.row(line, hd - H - G, pos);
    }
    float r = 1.f;
    if (hd < H + G && normalize && whole_norm && row_stat != nullptr) {
        r = row_stat[2 * n + (hd < H ? 0 : 1)];               // computed once per row by qk_row_stat_kernel
    } else if (hd < H + G && normalize) {
        // whole_norm: the statistic runs over all heads of the projection (queries: H * D values, keys: G * D) and the
        // weight has that size; else over the head alone, with a weight of D values shared by the heads
        const T* stat = whole_norm ? (hd < H ? qkv + n * ld : qkv + n * ld + (long long)H * D) : src;
        const int cnt = whole_norm ? (hd < H ? H : G) * D : dim;
        float ss = 0.f;
        for (int i = lane; i < cnt; i += 32) {
            const float v = ldf(stat + i);
            ss += v * v;
        }
        ss = warp_sum(ss);
        r = 1.f / sqrtf(ss / (float)cnt + eps);
    }
    // writeback: the normalised keys also replace the raw ones in the projection buffer, so that a kernel that reads
    // q / k / v as strided views of that buffer (prefill from position 0) sees what the cache holds
    T* back = (writeback && hd >= H && hd < H + G) ? const_cast<T*>(src) : nullptr;
    const float* wgt = hd < H ? q_weight : (hd < H + G ? k_weight : nullptr);
    if (wgt != nullptr && whole_norm) wgt += (long long)(hd < H ? hd : hd - H) * D;
    const int rot = (hd < H + G && rope_cos != nullptr) ? rope_dims : 0;
    // rotated part: pair i turns by the angle of (position, i); cos / sin come from a table [pos][i].  The pair is the
    // dimensions (2i, 2i + 1), or with rope_halves (i, i + rot / 2)
    if (rot > 0) {
        const long long pos = (long long)q_start[b] + t;
        const float* cs = rope_cos + pos * (rope_dims / 2);
        const float* sn = rope_sin + pos * (rope_dims / 2);
        for (int i = lane; i < rot / 2; i += 32) {
            const int iu = rope_halves ? i : 2 * i, iv = rope_halves ? i + rot / 2 : 2 * i + 1;
            float u = ldf(src + iu) * r, v = ldf(src + iv) * r;
            if (wgt != nullptr) {
                u *= wgt[iu];
                v *= wgt[iv];
            }
            const float c = cs[i], s = sn[i];
            stf(dst + iu, u * c - v * s);
            stf(dst + iv, v * c + u * s);
        }
    }
    for (int i = rot + lane; i < dim; i += 32) {
        float v = ldf(src + i) * r;
        if (wgt != nullptr) v *= wgt[i];
        stf(dst + i, v);
        if (back != nullptr) stf(back + i, v);
    }
}

// ---------------------------------------------------------------------------------------------------------------------
constexpr int BQ = 16, BK = 32, PF_THREADS = 128, MAXC = 64;   // MAXC * 8 = largest value size

template <typename T>
__global__ void __launch_bounds__(PF_THREADS)
window_attn_prefill_kernel(const T* __restrict__ q, const T* __restrict__ cache_k, const T* __restrict__ cache_v,
                           CacheAddr ka, CacheAddr va, T* __restrict__ out, const int* __restrict__ q_start,
                           const int* __restrict__ n_new, const int* __restrict__ seq_ids,
                           const float* __restrict__ slopes, int Tn, int H, int G, int D, int Dv, float scale, int window,
                           int keep_first, int chunk, const float* __restrict__ sinks) {
    extern __shared__ float smem[];
    float* Qs = smem;                       // [BQ][D]
    float* Ks = Qs + BQ * D;                // [BK][D + 1]
    float* Vs = Ks + BK * (D + 1);          // [BK][Dv]
    float* Ps = Vs + BK * Dv;               // [BQ][BK]
    __shared__ long long koff[BK], voff[BK];

    const int tid = threadIdx.x;
    const int q0 = blockIdx.x * BQ, h = blockIdx.y, b = blockIdx.z;
    const int g = h / (H / G);
    const int nb = n_new != nullptr ? min(n_new[b], Tn) : Tn;
    const int qi = tid >> 3, sub = tid & 7;
    const int nc = (Dv + 7) >> 3;
    T* orow = out + (((long long)b * Tn + q0 + qi) * H + h) * Dv;
    if (q0 >= nb) {                          // a tile of padding rows: defined output, no work
        if (q0 + qi < Tn)
            for (int m = 0; m < nc; ++m) {
                const int c = sub + 8 * m;
                if (c < Dv) stf(orow + c, 0.f);
            }
        return;
    }
    const int start = q_start[b];
    const int line = seq_ids != nullptr ? seq_ids[b] : b;
    const int p_lo = start + q0;
    const int p_hi = start + min(q0 + BQ, nb) - 1;
    const float slope = slopes != nullptr ? slopes[h] : 0.f;

    for (int idx = tid; idx < BQ * D; idx += PF_THREADS) {
        const int r = idx / D, c = idx - r * D;
        Qs[idx] = (q0 + r < nb) ? ldf(q + (((long long)b * Tn + q0 + r) * H + h) * D + c) * scale : 0.f;
    }
    const int p_i = start + q0 + qi;
    const bool row_ok = q0 + qi < nb;
    float m_i = -INFINITY, l_i = 0.f;
    float acc[MAXC];
#pragma unroll
    for (int m = 0; m < MAXC; ++m) acc[m] = 0.f;

    const int last_tile = p_hi / BK;
    for (int kt = 0; kt <= last_tile; ++kt) {
        const int k0 = kt * BK;
        if (window > 0 && k0 >= keep_first && k0 + BK - 1 <= p_lo - window) continue;   // nobody in the tile sees it
        if (chunk > 0 && k0 + BK - 1 < (p_lo / chunk) * chunk) continue;                 // before every query's chunk
        __syncthreads();                     // previous tile fully consumed (and Qs written, first time round)
        if (tid < BK) {
            const int pos = k0 + tid;
            koff[tid] = pos <= p_hi ? ka.row(line, g, pos) : -1;
            voff[tid] = pos <= p_hi ? va.row(line, g, pos) : -1;
        }
        __syncthreads();
        for (int idx = tid; idx < BK * D; idx += PF_THREADS) {
            const int r = idx / D, c = idx - r * D;
            Ks[r * (D + 1) + c] = koff[r] >= 0 ? ldf(cache_k + koff[r] + c) : 0.f;
        }
        for (int idx = tid; idx < BK * Dv; idx += PF_THREADS) {
            const int r = idx / Dv, c = idx - r * Dv;
            Vs[idx] = voff[r] >= 0 ? ldf(cache_v + voff[r] + c) : 0.f;
        }
        __syncthreads();
        float s[4];
        float tmax = -INFINITY;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int kj = sub + 8 * m;
            const int j = k0 + kj;
            const float* qr = Qs + qi * D;
            const float* kr = Ks + kj * (D + 1);
            float d = 0.f;
            for (int c = 0; c < D; ++c) d = fmaf(qr[c], kr[c], d);
            const int dist = p_i - j;
            const bool vis = row_ok && dist >= 0 && (window <= 0 || dist < window || j < keep_first) &&
                             (chunk <= 0 || p_i / chunk == j / chunk);
            s[m] = vis ? d - slope * (float)dist : -INFINITY;
            tmax = fmaxf(tmax, s[m]);
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
        const float m_new = fmaxf(m_i, tmax);
        const float alpha = (m_new == -INFINITY) ? 1.f : expf(m_i - m_new);
        float tsum = 0.f;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const float p = (s[m] == -INFINITY) ? 0.f : expf(s[m] - m_new);
            Ps[qi * BK + sub + 8 * m] = p;
            tsum += p;
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) tsum += __shfl_xor_sync(0xffffffffu, tsum, o);
        l_i = l_i * alpha + tsum;
        m_i = m_new;
        __syncwarp();                        // the 8 threads of a query row are lanes of one warp
        const float* pr = Ps + qi * BK;
#pragma unroll
        for (int m = 0; m < MAXC; ++m) {
            if (m < nc) {
                const int c = sub + 8 * m;
                float a = acc[m] * alpha;
                if (c < Dv) {
                    for (int kj = 0; kj < BK; ++kj) a = fmaf(pr[kj], Vs[kj * Dv + c], a);
                }
                acc[m] = a;
            }
        }
    }
    if (sinks != nullptr) l_i += expf(sinks[h] - (m_i == -INFINITY ? 0.f : m_i));
    if (q0 + qi < Tn) {
        const float inv = (row_ok && l_i > 0.f) ? 1.f / l_i : 0.f;
#pragma unroll
        for (int m = 0; m < MAXC; ++m) {
            if (m < nc) {
                const int c = sub + 8 * m;
                if (c < Dv) stf(orow + c, acc[m] * inv);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Tensor-core prefill for bf16 with compile-time head sizes (multiples of 16): 64 queries of one head per CTA (16 per
// warp, mma.sync m16n8k16), key / value tiles of 64 cache rows double-buffered with cp.async, rows padded by 16 bytes
// in shared memory (ldmatrix without bank conflicts for any D that is a multiple of 16), scores, bias, mask and the
// online softmax in fp32 registers, P handed to the PV product as A fragments without leaving registers.  The key
// tiles visited are the ones that hold kept first tokens plus the ones the window of some query of the tile reaches.
constexpr int MQ = 64, MK = 64, M_THREADS = 128;

template <int D, int DV>
__global__ void __launch_bounds__(M_THREADS)
window_attn_prefill_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ cache_k,
                               const bf16* __restrict__ cache_v, CacheAddr ka, CacheAddr va, bf16* __restrict__ out,
                               const int* __restrict__ q_start, const int* __restrict__ n_new,
                               const int* __restrict__ seq_ids, const float* __restrict__ slopes, int Tn, int H, int G,
                               float scale, int window, int keep_first, int chunk, const float* __restrict__ sinks) {
    constexpr int LDK = D + 8, LDV = DV + 8, CK = D / 8, CV = DV / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);       // [MQ][LDK]
    bf16* Ks = Qs + MQ * LDK;                           // [2][MK][LDK]
    bf16* Vs = Ks + 2 * MK * LDK;                       // [2][MK][LDV]
    __shared__ long long koff[2][MK], voff[2][MK];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int q0 = blockIdx.x * MQ, h = blockIdx.y, b = blockIdx.z;
    const int g = h / (H / G);
    const int nb = n_new != nullptr ? min(n_new[b], Tn) : Tn;
    if (q0 >= nb) {                                      // padding rows: zeros
        for (int idx = tid; idx < MQ * (DV / 2); idx += M_THREADS) {
            const int r = idx / (DV / 2), c = idx - r * (DV / 2);
            if (q0 + r < Tn)
                *reinterpret_cast<uint32_t*>(out + (((long long)b * Tn + q0 + r) * H + h) * DV + 2 * c) = 0u;
        }
        return;
    }
    const int start = q_start[b];
    const int line = seq_ids != nullptr ? seq_ids[b] : b;
    const int p_lo = start + q0;
    const int p_hi = start + min(q0 + MQ, nb) - 1;
    const int last_tile = p_hi / MK;
    int t_win = 0, n_sink_tiles = 0;
    if (window > 0) {
        t_win = max(0, p_lo - window + 1) / MK;
    }
    if (chunk > 0) t_win = max(t_win, ((p_lo / chunk) * chunk) / MK);     // tiles before the first query's chunk
    if (window > 0) n_sink_tiles = min((keep_first + MK - 1) / MK, t_win);
    const int n_tiles = n_sink_tiles + last_tile - t_win + 1;

    const uint32_t qs_addr = (uint32_t)__cvta_generic_to_shared(Qs);
    const uint32_t ks_addr = (uint32_t)__cvta_generic_to_shared(Ks);
    const uint32_t vs_addr = (uint32_t)__cvta_generic_to_shared(Vs);

    for (int idx = tid; idx < MQ * CK; idx += M_THREADS) {
        const int r = idx / CK, c = idx - r * CK;
        const bool ok = q0 + r < nb;
        const bf16* src = ok ? q + (((long long)b * Tn + q0 + r) * H + h) * D + c * 8 : q;
        mma::cp_async16(qs_addr + (r * LDK + c * 8) * 2, src, ok);
    }
    auto issue = [&](int n, int buf) {
        const int kt = n < n_sink_tiles ? n : t_win + (n - n_sink_tiles);
        if (tid < MK) {
            const int pos = kt * MK + tid;
            koff[buf][tid] = pos <= p_hi ? ka.row(line, g, pos) : -1;
        } else if (tid < 2 * MK) {
            const int pos = kt * MK + tid - MK;
            voff[buf][tid - MK] = pos <= p_hi ? va.row(line, g, pos) : -1;
        }
        __syncthreads();
        for (int idx = tid; idx < MK * CK; idx += M_THREADS) {
            const int r = idx / CK, c = idx - r * CK;
            const bool ok = koff[buf][r] >= 0;
            mma::cp_async16(ks_addr + ((buf * MK + r) * LDK + c * 8) * 2, ok ? cache_k + koff[buf][r] + c * 8 : cache_k, ok);
        }
        for (int idx = tid; idx < MK * CV; idx += M_THREADS) {
            const int r = idx / CV, c = idx - r * CV;
            const bool ok = voff[buf][r] >= 0;
            mma::cp_async16(vs_addr + ((buf * MK + r) * LDV + c * 8) * 2, ok ? cache_v + voff[buf][r] + c * 8 : cache_v, ok);
        }
        mma::cp_async_commit();
    };
    issue(0, 0);                                          // one group: the Q tile and the first K/V tile

    constexpr float LOG2E = 1.4426950408889634f;
    const float sc2 = scale * LOG2E;
    const float sl2 = (slopes != nullptr ? slopes[h] : 0.f) * LOG2E;
    const int r_lo = warp * 16 + (lane >> 2);             // this thread's rows: r_lo and r_lo + 8
    const int pi0 = start + q0 + r_lo, pi1 = pi0 + 8;
    const bool ok0 = q0 + r_lo < nb, ok1 = q0 + r_lo + 8 < nb;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    uint32_t qf[D / 16][4];

    for (int n = 0; n < n_tiles; ++n) {
        const int buf = n & 1;
        if (n + 1 < n_tiles) {
            issue(n + 1, buf ^ 1);
            mma::cp_async_wait<1>();
        } else {
            mma::cp_async_wait<0>();
        }
        __syncthreads();
        if (n == 0) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk)
                mma::ldsm_x4(qf[kk], qs_addr + ((warp * 16 + (lane & 15)) * LDK + kk * 16 + (lane >> 4) * 8) * 2);
        }
        const int kt = n < n_sink_tiles ? n : t_win + (n - n_sink_tiles);
        const int k0 = kt * MK;
        float s[MK / 8][4];
#pragma unroll
        for (int i = 0; i < MK / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
        const uint32_t kb_addr = ks_addr + buf * MK * LDK * 2;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
            for (int np = 0; np < MK / 16; ++np) {
                uint32_t bfr[4];
                const int row = np * 16 + (lane & 7) + (lane >> 4) * 8;
                mma::ldsm_x4(bfr, kb_addr + (row * LDK + kk * 16 + ((lane >> 3) & 1) * 8) * 2);
                mma::mma16816(s[2 * np], qf[kk], bfr[0], bfr[1]);
                mma::mma16816(s[2 * np + 1], qf[kk], bfr[2], bfr[3]);
            }
        }
        // scale, distance bias, mask; row maxima.  A tile that every query of the CTA sees completely needs no mask.
        float mx0 = -INFINITY, mx1 = -INFINITY;
        const bool full = q0 + MQ <= nb && k0 + MK - 1 <= p_lo &&
                          (window <= 0 || p_hi - k0 < window || k0 + MK <= keep_first) &&
                          (chunk <= 0 || k0 / chunk == p_hi / chunk);
        if (full) {
            const float jb = (float)(k0 + (lane & 3) * 2);
            const float c0 = sl2 * (jb - (float)pi0), c1 = sl2 * (jb - (float)pi1);     // -slope * (i - j) at column 0
#pragma unroll
            for (int i = 0; i < MK / 8; ++i) {
                const float d = sl2 * (float)(i * 8);
                s[i][0] = fmaf(s[i][0], sc2, c0 + d);
                s[i][1] = fmaf(s[i][1], sc2, c0 + d + sl2);
                s[i][2] = fmaf(s[i][2], sc2, c1 + d);
                s[i][3] = fmaf(s[i][3], sc2, c1 + d + sl2);
                mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
                mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
            }
        } else {
#pragma unroll
            for (int i = 0; i < MK / 8; ++i) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = k0 + i * 8 + (lane & 3) * 2 + (e & 1);
                    const int pi = (e & 2) ? pi1 : pi0;
                    const int dist = pi - j;
                    const bool vis = ((e & 2) ? ok1 : ok0) && dist >= 0 &&
                                     (window <= 0 || dist < window || j < keep_first) &&
                                     (chunk <= 0 || pi / chunk == j / chunk);
                    const float v = vis ? s[i][e] * sc2 - sl2 * (float)dist : -INFINITY;
                    s[i][e] = v;
                    if (e & 2) mx1 = fmaxf(mx1, v); else mx0 = fmaxf(mx0, v);
                }
            }
        }
        mx0 = mma::quad_max(mx0);
        mx1 = mma::quad_max(mx1);
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
        const float a0 = exp2f(m0 - ms0), a1 = exp2f(m1 - ms1);
        m0 = mn0;
        m1 = mn1;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int i = 0; i < MK / 8; ++i) {
            s[i][0] = exp2f(s[i][0] - ms0);
            s[i][1] = exp2f(s[i][1] - ms0);
            s[i][2] = exp2f(s[i][2] - ms1);
            s[i][3] = exp2f(s[i][3] - ms1);
            ps0 += s[i][0] + s[i][1];
            ps1 += s[i][2] + s[i][3];
        }
        l0 = l0 * a0 + ps0;
        l1 = l1 * a1 + ps1;
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) {
            o[i][0] *= a0;
            o[i][1] *= a0;
            o[i][2] *= a1;
            o[i][3] *= a1;
        }
        const uint32_t vb_addr = vs_addr + buf * MK * LDV * 2;
#pragma unroll
        for (int kb = 0; kb < MK / 16; ++kb) {
            uint32_t pa[4];
            pa[0] = mma::pack2(s[2 * kb][0], s[2 * kb][1]);
            pa[1] = mma::pack2(s[2 * kb][2], s[2 * kb][3]);
            pa[2] = mma::pack2(s[2 * kb + 1][0], s[2 * kb + 1][1]);
            pa[3] = mma::pack2(s[2 * kb + 1][2], s[2 * kb + 1][3]);
#pragma unroll
            for (int dj = 0; dj < DV / 16; ++dj) {
                uint32_t bfr[4];
                const int row = kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                mma::ldsm_x4_t(bfr, vb_addr + (row * LDV + dj * 16 + (lane >> 4) * 8) * 2);
                mma::mma16816(o[2 * dj], pa, bfr[0], bfr[1]);
                mma::mma16816(o[2 * dj + 1], pa, bfr[2], bfr[3]);
            }
        }
        __syncthreads();                                  // the buffer is free for the tile after next
    }
    l0 = mma::quad_sum(l0);
    l1 = mma::quad_sum(l1);
    if (sinks != nullptr) {
        const float sk = sinks[h] * LOG2E;
        l0 += exp2f(sk - (m0 == -INFINITY ? 0.f : m0));
        l1 += exp2f(sk - (m1 == -INFINITY ? 0.f : m1));
    }
    const float i0 = (ok0 && l0 > 0.f) ? 1.f / l0 : 0.f, i1 = (ok1 && l1 > 0.f) ? 1.f / l1 : 0.f;
    bf16* out0 = out + (((long long)b * Tn + q0 + r_lo) * H + h) * DV + (lane & 3) * 2;
    bf16* out1 = out0 + (long long)8 * H * DV;
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) {
        if (q0 + r_lo < Tn) *reinterpret_cast<uint32_t*>(out0 + i * 8) = mma::pack2(o[i][0] * i0, o[i][1] * i0);
        if (q0 + r_lo + 8 < Tn) *reinterpret_cast<uint32_t*>(out1 + i * 8) = mma::pack2(o[i][2] * i1, o[i][3] * i1);
    }
}

template <int D, int DV>
int launch_prefill_mma(const void* q, const void* ck, const void* cv, CacheAddr ka, CacheAddr va, void* out,
                       const int* q_start, const int* n_new, const int* seq_ids, const float* slopes, int B, int Tn, int H,
                       int G, float scale, int window, int keep_first, int chunk, const float* sinks, cudaStream_t st) {
    const size_t smem = (size_t)(MQ * (D + 8) + 2 * MK * (D + 8) + 2 * MK * (DV + 8)) * sizeof(bf16);
    auto kern = window_attn_prefill_mma_kernel<D, DV>;
    if (smem > 32 * 1024) NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((Tn + MQ - 1) / MQ, H, B);
    kern<<<grid, M_THREADS, smem, st>>>((const bf16*)q, (const bf16*)ck, (const bf16*)cv, ka, va, (bf16*)out, q_start,
                                        n_new, seq_ids, slopes, Tn, H, G, scale, window, keep_first, chunk, sinks);
    NXD_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
constexpr int DEC_WARPS = 8;   // DEC_R query heads per CTA, DEC_MV value columns per lane (Dv <= 32 * DEC_MV)

template <typename T, int DEC_R, int DEC_MV>
__global__ void __launch_bounds__(DEC_WARPS * 32)
window_attn_decode_kernel(const T* __restrict__ q, const T* __restrict__ cache_k, const T* __restrict__ cache_v,
                          CacheAddr ka, CacheAddr va, T* __restrict__ out, const int* __restrict__ positions,
                          const int* __restrict__ seq_ids, const float* __restrict__ slopes, int H, int G, int D, int Dv,
                          float scale, int window, int keep_first, int chunk, const float* __restrict__ sinks,
                          int groups_per_kv) {
    extern __shared__ float smem[];
    const int R_all = H / G;
    const int g = blockIdx.x / groups_per_kv, sub_group = blockIdx.x % groups_per_kv;
    const int b = blockIdx.y;
    const int r0 = sub_group * DEC_R;
    const int R = min(DEC_R, R_all - r0);
    const int h0 = g * R_all + r0;
    float* Qs = smem;                                   // [DEC_R][D]
    float* Ms = Qs + DEC_R * D;                         // [DEC_WARPS][DEC_R][Dv + 2]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int p = positions[b];
    const int line = seq_ids != nullptr ? seq_ids[b] : b;
    for (int idx = tid; idx < R * D; idx += DEC_WARPS * 32) {
        const int r = idx / D, c = idx - r * D;
        Qs[idx] = ldf(q + ((long long)b * H + h0 + r) * D + c) * scale;
    }
    __syncthreads();
    const int c_lo = chunk > 0 ? (p / chunk) * chunk : 0;          // first position of the query's chunk
    const int lo = max(window > 0 ? max(0, p - window + 1) : 0, c_lo);
    const int n_sink = max(0, min(keep_first, lo) - c_lo);         // kept first tokens below the window, inside the chunk
    const int nk = n_sink + (p - lo + 1);
    float m_r[DEC_R], l_r[DEC_R], sl[DEC_R];
    float acc[DEC_R][DEC_MV];
#pragma unroll
    for (int r = 0; r < DEC_R; ++r) {
        m_r[r] = -INFINITY;
        l_r[r] = 0.f;
        sl[r] = (slopes != nullptr && r < R) ? slopes[h0 + r] : 0.f;
#pragma unroll
        for (int m = 0; m < DEC_MV; ++m) acc[r][m] = 0.f;
    }
    for (int i = warp; i < nk; i += DEC_WARPS) {
        const int j = i < n_sink ? c_lo + i : lo + (i - n_sink);
        const T* kr = cache_k + ka.row(line, g, j);
        const T* vr = cache_v + va.row(line, g, j);
        float d[DEC_R];
#pragma unroll
        for (int r = 0; r < DEC_R; ++r) d[r] = 0.f;
        for (int c = lane; c < D; c += 32) {
            const float kv = ldf(kr + c);
#pragma unroll
            for (int r = 0; r < DEC_R; ++r)
                if (r < R) d[r] = fmaf(Qs[r * D + c], kv, d[r]);
        }
        float vv[DEC_MV];
#pragma unroll
        for (int m = 0; m < DEC_MV; ++m) {
            const int c = lane + 32 * m;
            vv[m] = c < Dv ? ldf(vr + c) : 0.f;
        }
        const float dist = (float)(p - j);
#pragma unroll
        for (int r = 0; r < DEC_R; ++r) {
            if (r < R) {
                const float s = warp_sum(d[r]) - sl[r] * dist;
                const float m_new = fmaxf(m_r[r], s);
                const float alpha = expf(m_r[r] - m_new);      // exp(-inf) = 0 on the first key
                const float pw = expf(s - m_new);
                l_r[r] = l_r[r] * alpha + pw;
                m_r[r] = m_new;
#pragma unroll
                for (int m = 0; m < DEC_MV; ++m) acc[r][m] = fmaf(pw, vv[m], acc[r][m] * alpha);
            }
        }
    }
    const int stride = Dv + 2;
#pragma unroll
    for (int r = 0; r < DEC_R; ++r) {
        if (r < R) {
            float* dst = Ms + ((long long)warp * DEC_R + r) * stride;
#pragma unroll
            for (int m = 0; m < DEC_MV; ++m) {
                const int c = lane + 32 * m;
                if (c < Dv) dst[c] = acc[r][m];
            }
            if (lane == 0) {
                dst[Dv] = m_r[r];
                dst[Dv + 1] = l_r[r];
            }
        }
    }
    __syncthreads();
    for (int idx = tid; idx < R * Dv; idx += DEC_WARPS * 32) {
        const int r = idx / Dv, c = idx - r * Dv;
        float mx = -INFINITY;
        for (int w = 0; w < DEC_WARPS; ++w) mx = fmaxf(mx, Ms[((long long)w * DEC_R + r) * stride + Dv]);
        float num = 0.f, den = 0.f;
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float* src = Ms + ((long long)w * DEC_R + r) * stride;
            const float mw = src[Dv];
            if (mw == -INFINITY) continue;
            const float f = expf(mw - mx);
            num = fmaf(f, src[c], num);
            den = fmaf(f, src[Dv + 1], den);
        }
        if (sinks != nullptr) den += expf(sinks[h0 + r] - (mx == -INFINITY ? 0.f : mx));
        stf(out + ((long long)b * H + h0 + r) * Dv + c, den > 0.f ? num / den : 0.f);
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Tensor-core decode for bf16: the (up to 16) query heads that share one key/value head are the 16 rows of the
// mma.sync tiles, so a cache row is read once for the whole group.  One CTA per (row, key/value head): the visible
// cache rows (kept first tokens, then the window) stream through the same double-buffered 64-row tiles as in prefill;
// each of the four warps takes 16 rows of a tile and keeps its own online-softmax state, merged through shared memory.
constexpr int DM_THREADS = 128, DM_ROWS = 16;

// VS: value columns per CTA.  A wide value row (the latent rows of a compressed key/value projection) is split over
// gridDim.z CTAs: each recomputes the scores of its 16 query heads and accumulates its own VS output columns, so the
// accumulator stays in registers; the other slices' reads of the same key rows hit L2.  QS: the query fragments are
// re-read from shared memory at every step of the key dimension instead of living in registers (large D).
template <int D, int DV, int VS, bool QS>
__global__ void __launch_bounds__(DM_THREADS)
window_attn_decode_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ cache_k,
                              const bf16* __restrict__ cache_v, CacheAddr ka, CacheAddr va, bf16* __restrict__ out,
                              const int* __restrict__ positions, const int* __restrict__ seq_ids,
                              const float* __restrict__ slopes, int H, int G, float scale, int window, int keep_first,
                              int chunk, const float* __restrict__ sinks, int groups_per_kv) {
    constexpr int LDK = D + 8, LDV = VS + 8, CK = D / 8, CV = VS / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);       // [DM_ROWS][LDK]
    bf16* Ks = Qs + DM_ROWS * LDK;                      // [2][MK][LDK]
    bf16* Vs = Ks + 2 * MK * LDK;                       // [2][MK][LDV]
    __shared__ long long koff[2][MK], voff[2][MK];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int R_all = H / G;
    const int g = blockIdx.x / groups_per_kv, r_base = (blockIdx.x % groups_per_kv) * DM_ROWS;
    const int b = blockIdx.y;
    const int vz = blockIdx.z * VS;                       // first value column of this CTA
    const int R = min(DM_ROWS, R_all - r_base);
    const int h0 = g * R_all + r_base;
    const int p = positions[b];
    const int line = seq_ids != nullptr ? seq_ids[b] : b;
    const int last_tile = p / MK;
    int t_win = 0, n_sink_tiles = 0;
    if (window > 0) {
        t_win = max(0, p - window + 1) / MK;
    }
    if (chunk > 0) t_win = max(t_win, ((p / chunk) * chunk) / MK);
    if (window > 0) n_sink_tiles = min((keep_first + MK - 1) / MK, t_win);
    const int n_tiles = n_sink_tiles + last_tile - t_win + 1;
    const uint32_t qs_addr = (uint32_t)__cvta_generic_to_shared(Qs);
    const uint32_t ks_addr = (uint32_t)__cvta_generic_to_shared(Ks);
    const uint32_t vs_addr = (uint32_t)__cvta_generic_to_shared(Vs);

    for (int idx = tid; idx < DM_ROWS * CK; idx += DM_THREADS) {
        const int r = idx / CK, c = idx - r * CK;
        const bool ok = r < R;
        mma::cp_async16(qs_addr + (r * LDK + c * 8) * 2, ok ? q + ((long long)b * H + h0 + r) * D + c * 8 : q, ok);
    }
    auto issue = [&](int n, int buf) {
        const int kt = n < n_sink_tiles ? n : t_win + (n - n_sink_tiles);
        if (tid < MK) {
            const int pos = kt * MK + tid;
            koff[buf][tid] = pos <= p ? ka.row(line, g, pos) : -1;
        } else {
            const int pos = kt * MK + tid - MK;
            voff[buf][tid - MK] = pos <= p ? va.row(line, g, pos) : -1;
        }
        __syncthreads();
        for (int idx = tid; idx < MK * CK; idx += DM_THREADS) {
            const int r = idx / CK, c = idx - r * CK;
            const bool ok = koff[buf][r] >= 0;
            mma::cp_async16(ks_addr + ((buf * MK + r) * LDK + c * 8) * 2, ok ? cache_k + koff[buf][r] + c * 8 : cache_k, ok);
        }
        for (int idx = tid; idx < MK * CV; idx += DM_THREADS) {
            const int r = idx / CV, c = idx - r * CV;
            const bool ok = voff[buf][r] >= 0;
            mma::cp_async16(vs_addr + ((buf * MK + r) * LDV + c * 8) * 2, ok ? cache_v + voff[buf][r] + vz + c * 8 : cache_v, ok);
        }
        mma::cp_async_commit();
    };
    issue(0, 0);

    constexpr float LOG2E = 1.4426950408889634f;
    const float sc2 = scale * LOG2E;
    const int r_lo = lane >> 2;                           // this thread's rows (query heads): r_lo and r_lo + 8
    const bool ok0 = r_lo < R, ok1 = r_lo + 8 < R;
    const float sl0 = (slopes != nullptr && ok0 ? slopes[h0 + r_lo] : 0.f) * LOG2E;
    const float sl1 = (slopes != nullptr && ok1 ? slopes[h0 + r_lo + 8] : 0.f) * LOG2E;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[VS / 8][4];
#pragma unroll
    for (int i = 0; i < VS / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    uint32_t qf[QS ? 1 : D / 16][4];

    for (int n = 0; n < n_tiles; ++n) {
        const int buf = n & 1;
        if (n + 1 < n_tiles) {
            issue(n + 1, buf ^ 1);
            mma::cp_async_wait<1>();
        } else {
            mma::cp_async_wait<0>();
        }
        __syncthreads();
        if (!QS && n == 0) {
#pragma unroll
            for (int kk = 0; kk < (QS ? 1 : D / 16); ++kk)
                mma::ldsm_x4(qf[kk], qs_addr + ((lane & 15) * LDK + kk * 16 + (lane >> 4) * 8) * 2);
        }
        const int kt = n < n_sink_tiles ? n : t_win + (n - n_sink_tiles);
        const int k0 = kt * MK + warp * 16;               // this warp's 16 cache rows of the tile
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
        const uint32_t kb_addr = ks_addr + buf * MK * LDK * 2;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            uint32_t bfr[4];
            const int row = warp * 16 + (lane & 7) + (lane >> 4) * 8;
            mma::ldsm_x4(bfr, kb_addr + (row * LDK + kk * 16 + ((lane >> 3) & 1) * 8) * 2);
            if (QS) mma::ldsm_x4(qf[0], qs_addr + ((lane & 15) * LDK + kk * 16 + (lane >> 4) * 8) * 2);
            mma::mma16816(s[0], qf[QS ? 0 : kk], bfr[0], bfr[1]);
            mma::mma16816(s[1], qf[QS ? 0 : kk], bfr[2], bfr[3]);
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = k0 + i * 8 + (lane & 3) * 2 + (e & 1);
                const int dist = p - j;
                const bool vis = ((e & 2) ? ok1 : ok0) && dist >= 0 &&
                                 (window <= 0 || dist < window || j < keep_first) && (chunk <= 0 || p / chunk == j / chunk);
                const float v = vis ? s[i][e] * sc2 - ((e & 2) ? sl1 : sl0) * (float)dist : -INFINITY;
                s[i][e] = v;
                if (e & 2) mx1 = fmaxf(mx1, v); else mx0 = fmaxf(mx0, v);
            }
        }
        mx0 = mma::quad_max(mx0);
        mx1 = mma::quad_max(mx1);
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
        const float a0 = exp2f(m0 - ms0), a1 = exp2f(m1 - ms1);
        m0 = mn0;
        m1 = mn1;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            s[i][0] = exp2f(s[i][0] - ms0);
            s[i][1] = exp2f(s[i][1] - ms0);
            s[i][2] = exp2f(s[i][2] - ms1);
            s[i][3] = exp2f(s[i][3] - ms1);
            ps0 += s[i][0] + s[i][1];
            ps1 += s[i][2] + s[i][3];
        }
        l0 = l0 * a0 + ps0;
        l1 = l1 * a1 + ps1;
        uint32_t pa[4];
        pa[0] = mma::pack2(s[0][0], s[0][1]);
        pa[1] = mma::pack2(s[0][2], s[0][3]);
        pa[2] = mma::pack2(s[1][0], s[1][1]);
        pa[3] = mma::pack2(s[1][2], s[1][3]);
        const uint32_t vb_addr = vs_addr + buf * MK * LDV * 2;
#pragma unroll
        for (int dj = 0; dj < VS / 16; ++dj) {
            uint32_t bfr[4];
            const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            mma::ldsm_x4_t(bfr, vb_addr + (row * LDV + dj * 16 + (lane >> 4) * 8) * 2);
            o[2 * dj][0] *= a0;
            o[2 * dj][1] *= a0;
            o[2 * dj][2] *= a1;
            o[2 * dj][3] *= a1;
            o[2 * dj + 1][0] *= a0;
            o[2 * dj + 1][1] *= a0;
            o[2 * dj + 1][2] *= a1;
            o[2 * dj + 1][3] *= a1;
            mma::mma16816(o[2 * dj], pa, bfr[0], bfr[1]);
            mma::mma16816(o[2 * dj + 1], pa, bfr[2], bfr[3]);
        }
        __syncthreads();
    }
    // merge the four warps: [warp][row][DV + 2] floats over the (now idle) tile buffers
    l0 = mma::quad_sum(l0);
    l1 = mma::quad_sum(l1);
    float* Ms = reinterpret_cast<float*>(smem_raw);
    constexpr int MS = VS + 2;
    {
        float* d0 = Ms + ((warp * DM_ROWS) + r_lo) * MS;
        float* d1 = d0 + 8 * MS;
#pragma unroll
        for (int i = 0; i < VS / 8; ++i) {
            const int c = i * 8 + (lane & 3) * 2;
            d0[c] = o[i][0];
            d0[c + 1] = o[i][1];
            d1[c] = o[i][2];
            d1[c + 1] = o[i][3];
        }
        if ((lane & 3) == 0) {
            d0[VS] = m0;
            d0[VS + 1] = l0;
            d1[VS] = m1;
            d1[VS + 1] = l1;
        }
    }
    __syncthreads();
    for (int idx = tid; idx < R * VS; idx += DM_THREADS) {
        const int r = idx / VS, c = idx - r * VS;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mx = fmaxf(mx, Ms[(w * DM_ROWS + r) * MS + VS]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float* src = Ms + (w * DM_ROWS + r) * MS;
            const float f = src[VS] == -INFINITY ? 0.f : exp2f(src[VS] - mx);
            num = fmaf(f, src[c], num);
            den = fmaf(f, src[VS + 1], den);
        }
        if (sinks != nullptr) den += exp2f(sinks[h0 + r] * LOG2E - (mx == -INFINITY ? 0.f : mx));
        out[((long long)b * H + h0 + r) * DV + vz + c] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
    }
}

template <int D, int DV, int VS = DV>
int launch_decode_mma(const void* q, const void* ck, const void* cv, CacheAddr ka, CacheAddr va, void* out,
                      const int* positions, const int* seq_ids, const float* slopes, int B, int H, int G, float scale,
                      int window, int keep_first, int chunk, const float* sinks, cudaStream_t st) {
    const int groups = (H / G + DM_ROWS - 1) / DM_ROWS;
    static_assert(DV % VS == 0 && VS % 16 == 0, "value slices");
    const size_t smem = (size_t)(DM_ROWS * (D + 8) + 2 * MK * (D + 8) + 2 * MK * (VS + 8)) * sizeof(bf16);
    auto kern = window_attn_decode_mma_kernel<D, DV, VS, (D > 256)>;
    if (smem > 32 * 1024) NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(G * groups, B, DV / VS);
    kern<<<grid, DM_THREADS, smem, st>>>((const bf16*)q, (const bf16*)ck, (const bf16*)cv, ka, va, (bf16*)out, positions,
                                         seq_ids, slopes, H, G, scale, window, keep_first, chunk, sinks, groups);
    NXD_LAUNCH_CHECK();
    return 0;
}

// maps [N, 2H, Dv]: heads 0 .. H-1 are the first attention map, H .. 2H-1 the second (same values).  One warp per
// (token, head): o = a1 - lambda a2 in fp32, divided by its root mean square over Dv, times (1 - diff).
template <typename T>
__global__ void diff_attn_combine_kernel(const T* __restrict__ maps, T* __restrict__ out, const float* __restrict__ lq1,
                                         const float* __restrict__ lk1, const float* __restrict__ lq2,
                                         const float* __restrict__ lk2, long long units, int H, int Dv, int D, float diff,
                                         float eps) {
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= units) return;
    float s1 = 0.f, s2 = 0.f;
    for (int i = lane; i < D; i += 32) {
        s1 = fmaf(lq1[i], lk1[i], s1);
        s2 = fmaf(lq2[i], lk2[i], s2);
    }
    const float lambda = expf(warp_sum(s1)) - expf(warp_sum(s2)) + diff;
    const long long n = unit / H;
    const int hd = (int)(unit % H);
    const T* a1 = maps + (n * 2 * H + hd) * Dv;
    const T* a2 = a1 + (long long)H * Dv;
    float ss = 0.f;
    for (int c = lane; c < Dv; c += 32) {
        const float o = ldf(a1 + c) - lambda * ldf(a2 + c);
        ss = fmaf(o, o, ss);
    }
    const float r = (1.f - diff) / sqrtf(warp_sum(ss) / (float)Dv + eps);
    T* dst = out + unit * Dv;
    for (int c = lane; c < Dv; c += 32) stf(dst + c, (ldf(a1 + c) - lambda * ldf(a2 + c)) * r);
}

CacheAddr make_addr(long long stride_line, long long stride_head, const int* block_table, int page_size, int table_cols,
                    int row_dim, int head_mod = 0) {
    CacheAddr a;
    a.head_mod = head_mod;
    a.stride_line = stride_line;
    a.stride_head = stride_head;
    a.block_table = block_table;
    a.page_size = page_size > 0 ? page_size : 1;
    a.table_cols = table_cols;
    a.row_dim = row_dim;
    return a;
}

template <typename T>
int launch_prefill(const void* q, const void* ck, const void* cv, CacheAddr ka, CacheAddr va, void* out,
                   const int* q_start, const int* n_new, const int* seq_ids, const float* slopes, int B, int Tn, int H,
                   int G, int D, int Dv, float scale, int window, int keep_first, int chunk, const float* sinks,
                   cudaStream_t st) {
    const size_t smem = (size_t)(BQ * D + BK * (D + 1) + BK * Dv + BQ * BK) * sizeof(float);
    auto kern = window_attn_prefill_kernel<T>;
    if (smem > 32 * 1024) NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((Tn + BQ - 1) / BQ, H, B);
    kern<<<grid, PF_THREADS, smem, st>>>((const T*)q, (const T*)ck, (const T*)cv, ka, va, (T*)out, q_start, n_new,
                                         seq_ids, slopes, Tn, H, G, D, Dv, scale, window, keep_first, chunk, sinks);
    NXD_LAUNCH_CHECK();
    return 0;
}

template <typename T, int DEC_R, int DEC_MV>
int launch_decode_rm(const void* q, const void* ck, const void* cv, CacheAddr ka, CacheAddr va, void* out,
                     const int* positions, const int* seq_ids, const float* slopes, int B, int H, int G, int D, int Dv,
                     float scale, int window, int keep_first, int chunk, const float* sinks, cudaStream_t st) {
    const int R_all = H / G;
    const int groups = (R_all + DEC_R - 1) / DEC_R;
    const size_t smem = (size_t)(DEC_R * D + DEC_WARPS * DEC_R * (Dv + 2)) * sizeof(float);
    auto kern = window_attn_decode_kernel<T, DEC_R, DEC_MV>;
    if (smem > 32 * 1024) NXD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(G * groups, B);
    kern<<<grid, DEC_WARPS * 32, smem, st>>>((const T*)q, (const T*)ck, (const T*)cv, ka, va, (T*)out, positions, seq_ids,
                                             slopes, H, G, D, Dv, scale, window, keep_first, chunk, sinks, groups);
    NXD_LAUNCH_CHECK();
    return 0;
}

template <typename T>
int launch_decode(const void* q, const void* ck, const void* cv, CacheAddr ka, CacheAddr va, void* out,
                  const int* positions, const int* seq_ids, const float* slopes, int B, int H, int G, int D, int Dv,
                  float scale, int window, int keep_first, int chunk, const float* sinks, cudaStream_t st) {
    if (Dv <= 256)
        return launch_decode_rm<T, 8, 8>(q, ck, cv, ka, va, out, positions, seq_ids, slopes, B, H, G, D, Dv, scale, window,
                                         keep_first, chunk, sinks, st);
    return launch_decode_rm<T, 4, 16>(q, ck, cv, ka, va, out, positions, seq_ids, slopes, B, H, G, D, Dv, scale, window,
                                      keep_first, chunk, sinks, st);      // wide value rows: fewer heads per CTA
}

}  // namespace

// dtype: 0 = bf16, 1 = fp32 (projection output, q, cache and attention output share it).  qkv: [B * Tn, ld] rows laid
// out as H query heads of D, then (has_kv) G key heads of D and G value heads of Dv.  q_start [B]: position of the first
// new token of every row; n_new [B] or NULL: how many of the Tn rows are real (the others are padding and write
// nothing); seq_ids [B] or NULL: cache line of every row.  max_pos: rows of a cache line.
// q_weight / k_weight [D] fp32 or NULL: weight of the per-head norm.  rope_cos / rope_sin [positions, rope_dims / 2]
// fp32 or NULL: queries and keys (after the norm) turn pairwise, (2i, 2i + 1), on their first rope_dims dimensions
// (rope_halves: the pairs are (i, i + rope_dims / 2)).  whole_norm: the norm's statistic runs over all query heads (all
// key heads) of a row at once and q_weight / k_weight hold H * D / G * D values; row_stat [B * Tn, 2] fp32 scratch (or NULL:
// every head's warp computes the row statistic itself).
// value_from_key: the row has no value columns, the cached value is the raw key projection (taken ahead of the norm and the rotation).
NXD_API int nxd_qk_prep_cache_write(int dtype, const void* qkv, long long ld, void* q_out, void* cache_k, void* cache_v,
                                    long long k_stride_line, long long k_stride_head, long long v_stride_line,
                                    long long v_stride_head, const int* block_table, int page_size, int table_cols,
                                    const int* q_start, const int* n_new, const int* seq_ids, int B, int Tn, int H, int G,
                                    int D, int Dv, int has_kv, int normalize, float eps, int max_pos, int writeback,
                                    const float* q_weight, const float* k_weight, const float* rope_cos,
                                    const float* rope_sin, int rope_dims, int value_from_key, int value_heads,
                                    int rope_halves, int whole_norm, float* row_stat, void* stream) {
    const int Gv = value_heads > 0 ? value_heads : G;
    const long long units = (long long)B * Tn * (H + (has_kv ? G + Gv : 0));
    if (units == 0) return 0;
    NXD_REQUIRE(!value_from_key || Gv == G, "values taken from the keys need as many value heads (%d) as key heads (%d)", Gv, G);
    NXD_REQUIRE(rope_cos == nullptr || (rope_dims % 2 == 0 && rope_dims <= D), "rotation over %d of %d dimensions", rope_dims, D);
    NXD_REQUIRE(!value_from_key || Dv == D, "values taken from the keys need equal sizes (%d, %d)", D, Dv);
    NXD_REQUIRE(!(writeback && rope_cos != nullptr), "write-back of rotated keys is not %s", "supported");
    const CacheAddr ka = make_addr(k_stride_line, k_stride_head, block_table, page_size, table_cols, D);
    const CacheAddr va = make_addr(v_stride_line, v_stride_head, block_table, page_size, table_cols, Dv);
    const int wpb = 8;
    const unsigned blocks = (unsigned)((units + wpb - 1) / wpb);
    if (!(whole_norm && normalize)) row_stat = nullptr;
    if (row_stat != nullptr) {           // the whole-projection statistics once per row, ahead of the per-head warps
        const long long rows = (long long)B * Tn;
        const unsigned sb = (unsigned)((rows + wpb - 1) / wpb);
        if (dtype == 0)
            qk_row_stat_kernel<bf16><<<sb, wpb * 32, 0, (cudaStream_t)stream>>>((const bf16*)qkv, ld, row_stat, rows, H * D,
                                                                                has_kv ? G * D : 0, eps);
        else
            qk_row_stat_kernel<float><<<sb, wpb * 32, 0, (cudaStream_t)stream>>>((const float*)qkv, ld, row_stat, rows, H * D,
                                                                                 has_kv ? G * D : 0, eps);
        NXD_LAUNCH_CHECK();
    }
    if (dtype == 0)
        qk_norm_cache_write_kernel<bf16><<<blocks, wpb * 32, 0, (cudaStream_t)stream>>>(
            (const bf16*)qkv, ld, (bf16*)q_out, (bf16*)cache_k, (bf16*)cache_v, ka, va, q_start, n_new, seq_ids, units, Tn,
            H, G, D, Dv, has_kv, normalize, eps, max_pos, writeback, q_weight, k_weight, rope_cos, rope_sin, rope_dims,
            value_from_key, Gv, rope_halves, whole_norm, row_stat);
    else
        qk_norm_cache_write_kernel<float><<<blocks, wpb * 32, 0, (cudaStream_t)stream>>>(
            (const float*)qkv, ld, (float*)q_out, (float*)cache_k, (float*)cache_v, ka, va, q_start, n_new, seq_ids, units,
            Tn, H, G, D, Dv, has_kv, normalize, eps, max_pos, writeback, q_weight, k_weight, rope_cos, rope_sin, rope_dims,
            value_from_key, Gv, rope_halves, whole_norm, row_stat);
    NXD_LAUNCH_CHECK();
    return 0;
}

NXD_API int nxd_qk_norm_cache_write(int dtype, const void* qkv, long long ld, void* q_out, void* cache_k, void* cache_v,
                                    long long k_stride_line, long long k_stride_head, long long v_stride_line,
                                    long long v_stride_head, const int* block_table, int page_size, int table_cols,
                                    const int* q_start, const int* n_new, const int* seq_ids, int B, int Tn, int H, int G,
                                    int D, int Dv, int has_kv, int normalize, float eps, int max_pos, int writeback,
                                    void* stream) {
    return nxd_qk_prep_cache_write(dtype, qkv, ld, q_out, cache_k, cache_v, k_stride_line, k_stride_head, v_stride_line,
                                   v_stride_head, block_table, page_size, table_cols, q_start, n_new, seq_ids, B, Tn, H, G,
                                   D, Dv, has_kv, normalize, eps, max_pos, writeback, nullptr, nullptr, nullptr, nullptr, 0,
                                   0, 0, 0, 0, nullptr, stream);
}

// q [B, Tn, H, D] -> out [B, Tn, H, Dv]; the keys and values of positions [0, q_start[b] + n_new[b]) are read from the
// cache (the new tokens' rows must have been written before).  slopes [H] fp32 or NULL; window <= 0: no window;
// chunk <= 0: no chunks; sinks [H] fp32 or NULL.  k_row / v_row: elements between consecutive cache rows (D / Dv for
// tensors of their own; v_row == k_row when the values are columns of the key rows).
// impl: 0 = choose, 1 = the generic kernel, 2 = the tensor-core kernel (an error when it does not apply).
NXD_API int nxd_masked_attn_prefill(int dtype, const void* q, const void* cache_k, const void* cache_v,
                                    long long k_stride_line, long long k_stride_head, long long k_row,
                                    long long v_stride_line, long long v_stride_head, long long v_row,
                                    const int* block_table, int page_size, int table_cols, void* out, const int* q_start,
                                    const int* n_new, const int* seq_ids, const float* slopes, const float* sinks, int B,
                                    int Tn, int H, int G, int D, int Dv, float scale, int window, int keep_first, int chunk,
                                    int impl, int value_heads, void* stream) {
    NXD_REQUIRE(G > 0 && H % G == 0, "attention: %d query heads over %d key/value heads", H, G);
    NXD_REQUIRE(Dv <= MAXC * 8, "attention: value size %d above %d", Dv, MAXC * 8);
    if (B * Tn == 0) return 0;
    const int vmod = (value_heads > 0 && value_heads < G) ? value_heads : 0;
    const CacheAddr ka = make_addr(k_stride_line, k_stride_head, block_table, page_size, table_cols, (int)k_row);
    const CacheAddr va = make_addr(v_stride_line, v_stride_head, block_table, page_size, table_cols, (int)v_row, vmod);
    cudaStream_t st = (cudaStream_t)stream;
    // bf16 with head sizes the tensor-core kernel is compiled for (cache rows must start on 16-byte boundaries);
    // everything else takes the generic kernel
    if (dtype == 0 && impl != 1 && Tn >= 16 && (k_stride_head % 8) == 0 && (v_stride_head % 8) == 0 &&
        (k_stride_line % 8) == 0 && (v_stride_line % 8) == 0 && (k_row % 8) == 0 && (v_row % 8) == 0 &&
        ((uintptr_t)cache_k % 16) == 0 && ((uintptr_t)cache_v % 16) == 0) {
#define NXD_WA_CASE(DD, DDV)                                                                                          \
    if (D == DD && Dv == DDV)                                                                                         \
        return launch_prefill_mma<DD, DDV>(q, cache_k, cache_v, ka, va, out, q_start, n_new, seq_ids, slopes, B, Tn, H, \
                                           G, scale, window, keep_first, chunk, sinks, st)
        NXD_WA_CASE(32, 32);
        NXD_WA_CASE(64, 64);
        NXD_WA_CASE(96, 96);
        NXD_WA_CASE(128, 128);
        NXD_WA_CASE(64, 128);
        NXD_WA_CASE(128, 64);
        NXD_WA_CASE(96, 64);      // key size = un-rotated + rotated dimensions of an expanded latent head
        NXD_WA_CASE(192, 128);
        NXD_WA_CASE(32, 64);      // two attention maps of half the value size (differential attention)
        NXD_WA_CASE(48, 96);
        NXD_WA_CASE(96, 192);
        NXD_WA_CASE(128, 256);
#undef NXD_WA_CASE
    }
    NXD_REQUIRE(impl != 2, "attention: no tensor-core kernel for bf16=%d D=%d Dv=%d", dtype == 0, D, Dv);
    if (dtype == 0)
        return launch_prefill<bf16>(q, cache_k, cache_v, ka, va, out, q_start, n_new, seq_ids, slopes, B, Tn, H, G, D, Dv,
                                    scale, window, keep_first, chunk, sinks, st);
    return launch_prefill<float>(q, cache_k, cache_v, ka, va, out, q_start, n_new, seq_ids, slopes, B, Tn, H, G, D, Dv,
                                 scale, window, keep_first, chunk, sinks, st);
}

NXD_API int nxd_window_attn_prefill(int dtype, const void* q, const void* cache_k, const void* cache_v,
                                    long long k_stride_line, long long k_stride_head, long long v_stride_line,
                                    long long v_stride_head, const int* block_table, int page_size, int table_cols,
                                    void* out, const int* q_start, const int* n_new, const int* seq_ids,
                                    const float* slopes, int B, int Tn, int H, int G, int D, int Dv, float scale,
                                    int window, int keep_first, int impl, void* stream) {
    return nxd_masked_attn_prefill(dtype, q, cache_k, cache_v, k_stride_line, k_stride_head, D, v_stride_line,
                                   v_stride_head, Dv, block_table, page_size, table_cols, out, q_start, n_new, seq_ids,
                                   slopes, nullptr, B, Tn, H, G, D, Dv, scale, window, keep_first, 0, impl, 0, stream);
}

// q [B, H, D] of one new token per row at positions[b] (its key and value already in the cache) -> out [B, H, Dv].
NXD_API int nxd_masked_attn_decode(int dtype, const void* q, const void* cache_k, const void* cache_v,
                                   long long k_stride_line, long long k_stride_head, long long k_row,
                                   long long v_stride_line, long long v_stride_head, long long v_row,
                                   const int* block_table, int page_size, int table_cols, void* out, const int* positions,
                                   const int* seq_ids, const float* slopes, const float* sinks, int B, int H, int G, int D,
                                   int Dv, float scale, int window, int keep_first, int chunk, int impl, int value_heads,
                                   void* stream) {
    NXD_REQUIRE(G > 0 && H % G == 0, "attention: %d query heads over %d key/value heads", H, G);
    NXD_REQUIRE(Dv <= 512, "attention: value size %d above %d", Dv, 512);
    if (B == 0) return 0;
    const int vmod = (value_heads > 0 && value_heads < G) ? value_heads : 0;
    const CacheAddr ka = make_addr(k_stride_line, k_stride_head, block_table, page_size, table_cols, (int)k_row);
    const CacheAddr va = make_addr(v_stride_line, v_stride_head, block_table, page_size, table_cols, (int)v_row, vmod);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == 0 && impl != 1 && (k_stride_head % 8) == 0 && (v_stride_head % 8) == 0 && (k_stride_line % 8) == 0 &&
        (v_stride_line % 8) == 0 && (k_row % 8) == 0 && (v_row % 8) == 0 && ((uintptr_t)cache_k % 16) == 0 &&
        ((uintptr_t)cache_v % 16) == 0) {
#define NXD_WD_CASE(DD, DDV)                                                                                          \
    if (D == DD && Dv == DDV)                                                                                         \
        return launch_decode_mma<DD, DDV>(q, cache_k, cache_v, ka, va, out, positions, seq_ids, slopes, B, H, G, scale, \
                                          window, keep_first, chunk, sinks, st)
        NXD_WD_CASE(32, 32);
        NXD_WD_CASE(64, 64);
        NXD_WD_CASE(96, 96);
        NXD_WD_CASE(128, 128);
        NXD_WD_CASE(64, 128);
        NXD_WD_CASE(128, 64);
        NXD_WD_CASE(160, 128);    // latent rows: compressed key/value + shared rotated key part; value = the compressed part
        NXD_WD_CASE(32, 64);      // two attention maps of half the value size (differential attention)
        NXD_WD_CASE(48, 96);
        NXD_WD_CASE(96, 192);
        NXD_WD_CASE(128, 256);
#undef NXD_WD_CASE
        if (D == 288 && Dv == 256)                   // wide latent rows: the value columns are split over CTAs
            return launch_decode_mma<288, 256, 128>(q, cache_k, cache_v, ka, va, out, positions, seq_ids, slopes, B, H, G,
                                                    scale, window, keep_first, chunk, sinks, st);
        if (D == 576 && Dv == 512)
            return launch_decode_mma<576, 512, 128>(q, cache_k, cache_v, ka, va, out, positions, seq_ids, slopes, B, H, G,
                                                    scale, window, keep_first, chunk, sinks, st);
    }
    NXD_REQUIRE(impl != 2, "attention decode: no tensor-core kernel for bf16=%d D=%d Dv=%d", dtype == 0, D, Dv);
    if (dtype == 0)
        return launch_decode<bf16>(q, cache_k, cache_v, ka, va, out, positions, seq_ids, slopes, B, H, G, D, Dv, scale,
                                   window, keep_first, chunk, sinks, st);
    return launch_decode<float>(q, cache_k, cache_v, ka, va, out, positions, seq_ids, slopes, B, H, G, D, Dv, scale,
                                window, keep_first, chunk, sinks, st);
}

NXD_API int nxd_window_attn_decode(int dtype, const void* q, const void* cache_k, const void* cache_v,
                                   long long k_stride_line, long long k_stride_head, long long v_stride_line,
                                   long long v_stride_head, const int* block_table, int page_size, int table_cols,
                                   void* out, const int* positions, const int* seq_ids, const float* slopes, int B, int H,
                                   int G, int D, int Dv, float scale, int window, int keep_first, int impl, void* stream) {
    return nxd_masked_attn_decode(dtype, q, cache_k, cache_v, k_stride_line, k_stride_head, D, v_stride_line,
                                  v_stride_head, Dv, block_table, page_size, table_cols, out, positions, seq_ids, slopes,
                                  nullptr, B, H, G, D, Dv, scale, window, keep_first, 0, impl, 0, stream);
}

NXD_API int nxd_diff_attn_combine(int dtype, const void* maps, void* out, const float* lq1, const float* lk1,
                                  const float* lq2, const float* lk2, long long N, int H, int Dv, int D, float diff,
                                  float eps, void* stream) {
    const long long units = N * H;
    if (units == 0) return 0;
    const int wpb = 8;
    const unsigned blocks = (unsigned)((units + wpb - 1) / wpb);
    if (dtype == 0)
        diff_attn_combine_kernel<bf16><<<blocks, wpb * 32, 0, (cudaStream_t)stream>>>((const bf16*)maps, (bf16*)out, lq1, lk1,
                                                                                     lq2, lk2, units, H, Dv, D, diff, eps);
    else
        diff_attn_combine_kernel<float><<<blocks, wpb * 32, 0, (cudaStream_t)stream>>>((const float*)maps, (float*)out, lq1,
                                                                                      lk1, lq2, lk2, units, H, Dv, D, diff,
                                                                                      eps);
    NXD_LAUNCH_CHECK();
    return 0;
}
