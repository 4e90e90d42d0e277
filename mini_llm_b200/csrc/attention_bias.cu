// Causal softmax attention over the paged cache with three things the plain kernels do not have:
//   * keys and values of different row sizes (dk for queries and keys, dv for values and outputs);
//   * an additive score bias that depends on the head and on the distance i - j only, given as a table
//     dist_bias[head][distance] (a logarithmic or linear distance penalty, say);
//   * a factor on the query that depends on its position only, given as a table q_scale[position]
//     (a query "temperature" that grows with the context).
// score(i, j) = (q_i . k_j) * scale * q_scale[i] + dist_bias[h][i - j] for j <= i (and j > i - window when a
// window is set); softmax over the visible keys; out_i = out_scale * sum_j p_ij v_j.  Either table may be absent.
// Scores, biases, softmax and the weighted sum are 32-bit (expf, not the fast intrinsic) for both cache dtypes.
//
// Three kernels.  `simt`: one warp per (token, head), 32 keys at a time: any step, and the plain twin of the
// others.  `tiled`: 64 queries x 32 keys per CTA and head for prompt portions: queries in shared memory, a key
// tile staged transposed and a value tile as it is, 2 x 4 scores and 2 x dv/8 outputs per thread.  `split`: single
// tokens (decode): the keys of a token are cut into splits of 256 starting at multiples of 256 from position 0, a
// CTA takes one split for up to four query heads that share a key/value head (rows staged once in shared memory),
// the partial (o, m, l) of the splits are merged in split order by a second kernel.  Key chunks and tiles start at multiples of 32 from position 0 in all three, so a token's
// sums run in an order that depends on its position only, not on how the step was cut or batched.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_D = 256;          // largest dk and dv

template <typename T>
__device__ __forceinline__ void load8(const T* p, float* f) {   // 8 consecutive elements (bfloat16) or 4 + 4 (float)
    if constexpr (sizeof(T) == 4) {
        const float4 a = *reinterpret_cast<const float4*>(p);
        const float4 b = *reinterpret_cast<const float4*>(p + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
        const uint4 u = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) { f[2 * i] = __low2float(b2[i]); f[2 * i + 1] = __high2float(b2[i]); }
    }
}

struct BiasArgs {
    const float* dist_bias;     // [H][n_dist] or null
    int n_dist;
    const float* q_scale;       // [n_pos] or null
    float scale, out_scale;
    int window;
};

// One warp walks the keys [k_lo, k_hi] (inclusive, absolute positions) of one (token, head) in chunks of 32 that
// start at multiples of 32, and leaves the online-softmax state: acc (lane d holds dims d, d+32, ...), m, l.
template <typename T>
__device__ __forceinline__ void warp_walk(const float* qs, const T* k_pages, const T* v_pages, const int* bt, int p, int h,
                                          int hk, int Hkv, int dk, int dv, int page_size, int k_lo, int k_hi,
                                          const BiasArgs& a, float qf, float* acc, float& m, float& l) {
    const int lane = threadIdx.x & 31;
    constexpr int NACC = MAX_D / 32;
    const float* brow = a.dist_bias ? a.dist_bias + (size_t)h * a.n_dist : nullptr;
    for (int c0 = (k_lo / 32) * 32; c0 <= k_hi; c0 += 32) {
        const int kp = c0 + lane;
        const bool valid = kp >= k_lo && kp <= k_hi;
        float s = -INFINITY;
        if (valid) {
            const int page = bt[kp / page_size];
            const T* kr = k_pages + (((size_t)page * Hkv + hk) * page_size + kp % page_size) * dk;
            float dot = 0.f;
            for (int d = 0; d < dk; d += 8) {
                float kv[8];
                load8(kr + d, kv);
#pragma unroll
                for (int i = 0; i < 8; ++i) dot = fmaf(qs[d + i], kv[i], dot);
            }
            s = dot * qf;
            if (brow) s += brow[p - kp];
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;                 // no key of the chunk is in the range (uniform)
        const float alpha = expf(m - m_new);
        const float pr = valid ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(pr);
        m = m_new;
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= alpha;
        const int j0 = max(0, k_lo - c0), j1 = min(32, k_hi - c0 + 1);
        for (int j = j0; j < j1; ++j) {
            const float pj = __shfl_sync(0xffffffffu, pr, j);
            const int kpj = c0 + j;
            const int page = bt[kpj / page_size];
            const T* vr = v_pages + (((size_t)page * Hkv + hk) * page_size + kpj % page_size) * dv;
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                const int d = lane + 32 * i;
                if (d < dv) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_bias_simt_kernel(const T* q, long long q_stride, const T* k_pages, const T* v_pages,
                           const int* __restrict__ block_table, int bt_stride, const int* __restrict__ token_seq,
                           const int* __restrict__ positions, T* __restrict__ out, long long out_stride, int T_tokens,
                           int H, int Hkv, int dk, int dv, int page_size, BiasArgs a) {
    __shared__ float qs[WARPS][MAX_D];
    pdl_wait();
    pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long gw = (long long)blockIdx.x * WARPS + warp;
    if (gw >= (long long)T_tokens * H) return;
    const int t = (int)(gw / H), h = (int)(gw % H);
    const int hk = h / (H / Hkv);
    const int seq = token_seq[t], p = positions[t];
    const int* bt = block_table + (size_t)seq * bt_stride;
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * dk;
    for (int d = lane; d < dk; d += 32) qs[warp][d] = to_f32(qrow[d]);
    __syncwarp();
    const float qf = a.scale * (a.q_scale ? a.q_scale[p] : 1.0f);
    int first = 0;
    if (a.window > 0 && p - a.window + 1 > 0) first = p - a.window + 1;
    constexpr int NACC = MAX_D / 32;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    warp_walk<T>(qs[warp], k_pages, v_pages, bt, p, h, hk, Hkv, dk, dv, page_size, first, p, a, qf, acc, m, l);
    T* orow = out + (size_t)t * out_stride + (size_t)h * dv;
    const float inv = a.out_scale / l;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) orow[d] = from_f32<T>(acc[i] * inv);
    }
}

// ------------------------------------------------------------------------------------------------ decode
constexpr int SPLIT = 256;          // keys per split

// Single tokens.  grid (splits, kv heads x head chunks, tokens).  A CTA takes one split of one token's keys for HG
// (1, 2 or 4) query heads that share a key/value head, so a key or value row is fetched once for all of them.  The
// split is walked in tiles of 32 * KS keys (KS = 4 / HG key sub-tiles) that are staged in shared memory with 16-byte
// loads (all loads of a burst before any store); warp w takes head w % HG and sub-tile w / HG: its lanes are the 32
// keys for the scores (a row of K per lane, the query broadcast) and 32 value columns at a time for the weighted sum.
// Sub-tile k of tile i covers the absolute positions [split*256 + (i*KS + k)*32, +32): chunks of 32 from position 0.
// Partial results: part_o [T][H][splits][dv], part_ml [T][H][splits][2]; a split without visible keys writes l = 0.
template <typename T>
__global__ void __launch_bounds__(128)
attention_bias_split_kernel(const T* q, long long q_stride, const T* k_pages, const T* v_pages,
                            const int* __restrict__ block_table, int bt_stride, const int* __restrict__ token_seq,
                            const int* __restrict__ positions, float* __restrict__ part_o, float* __restrict__ part_ml,
                            int H, int Hkv, int dk, int dv, int page_size, int HG, int KS, BiasArgs a) {
    extern __shared__ __align__(16) unsigned char smraw[];
    constexpr int VEC = 16 / sizeof(T);
    const int krow = dk + VEC;                                  // elements per staged key row: 16 bytes of padding
    const int tile = 32 * KS;
    T* Ks = reinterpret_cast<T*>(smraw);                        // [tile][dk + VEC]
    T* Vs = Ks + (size_t)tile * krow;                           // [tile][dv]
    float* qs = reinterpret_cast<float*>(Vs + (((size_t)tile * dv + VEC - 1) / VEC) * VEC);   // [HG][dk]
    float* so = qs + HG * dk;                                   // [warps][dv] at the end
    float* sml = so + 4 * dv;                                   // [warps][2]
    pdl_wait();
    pdl_launch();
    const int split = blockIdx.x, nsplit = gridDim.x, t = blockIdx.z;
    const int R = H / Hkv, chunks = (R + HG - 1) / HG;
    const int hk = blockIdx.y / chunks, h0 = hk * R + (blockIdx.y % chunks) * HG;
    const int nh = min(HG, hk * R + R - h0);                    // heads this CTA really has
    const int tid = threadIdx.x, nthreads = blockDim.x, warp = tid >> 5, lane = tid & 31;
    const int wh = warp % HG, wk = warp / HG;                   // this warp's head and key sub-tile
    const int h = h0 + wh;
    const bool live = wh < nh;
    const int seq = token_seq[t], p = positions[t];
    int first = 0;
    if (a.window > 0 && p - a.window + 1 > 0) first = p - a.window + 1;
    const int s_lo = max(first, split * SPLIT), s_hi = min(p, split * SPLIT + SPLIT - 1);
    if (s_lo > s_hi) {                                          // uniform over the CTA
        if (tid < nh) { const size_t pi = ((size_t)t * H + h0 + tid) * nsplit + split; part_ml[pi * 2] = -INFINITY; part_ml[pi * 2 + 1] = 0.f; }
        return;
    }
    const int* bt = block_table + (size_t)seq * bt_stride;
    for (int i = tid; i < HG * dk; i += nthreads) {
        const int hh = i / dk, d = i % dk;
        qs[i] = hh < nh ? to_f32(q[(size_t)t * q_stride + (size_t)(h0 + hh) * dk + d]) : 0.f;
    }
    const float qf = a.scale * (a.q_scale ? a.q_scale[p] : 1.0f);
    const float* brow = (a.dist_bias && live) ? a.dist_bias + (size_t)h * a.n_dist : nullptr;
    constexpr int NACC = MAX_D / 32;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int kpieces = dk / VEC;
    const int vpieces = (dv % VEC == 0 && ((uintptr_t)v_pages % 16) == 0) ? dv / VEC : 0;   // 0: value rows are copied by element

    for (int base = (s_lo / tile) * tile; base <= s_hi; base += tile) {
        __syncthreads();                                        // the tile before is no longer read; qs is complete
        constexpr int LD = 4;
        for (int i0 = tid; i0 < tile * kpieces; i0 += nthreads * LD) {
            uint4 r[LD];
#pragma unroll
            for (int u = 0; u < LD; ++u) {
                const int i = i0 + u * nthreads, key = i / kpieces, piece = i % kpieces, kp = base + key;
                r[u] = make_uint4(0u, 0u, 0u, 0u);
                if (i < tile * kpieces && kp >= s_lo && kp <= s_hi)
                    r[u] = *reinterpret_cast<const uint4*>(k_pages + (((size_t)bt[kp / page_size] * Hkv + hk) * page_size + kp % page_size) * dk + piece * VEC);
            }
#pragma unroll
            for (int u = 0; u < LD; ++u) {
                const int i = i0 + u * nthreads;
                if (i < tile * kpieces) *reinterpret_cast<uint4*>(Ks + (size_t)(i / kpieces) * krow + (i % kpieces) * VEC) = r[u];
            }
        }
        if (vpieces) {
            for (int i0 = tid; i0 < tile * vpieces; i0 += nthreads * LD) {
                uint4 r[LD];
#pragma unroll
                for (int u = 0; u < LD; ++u) {
                    const int i = i0 + u * nthreads, key = i / vpieces, piece = i % vpieces, kp = base + key;
                    r[u] = make_uint4(0u, 0u, 0u, 0u);
                    if (i < tile * vpieces && kp >= s_lo && kp <= s_hi)
                        r[u] = *reinterpret_cast<const uint4*>(v_pages + (((size_t)bt[kp / page_size] * Hkv + hk) * page_size + kp % page_size) * dv + piece * VEC);
                }
#pragma unroll
                for (int u = 0; u < LD; ++u) {
                    const int i = i0 + u * nthreads;
                    if (i < tile * vpieces) *reinterpret_cast<uint4*>(Vs + (size_t)(i / vpieces) * dv + (i % vpieces) * VEC) = r[u];
                }
            }
        } else {
            for (int i = tid; i < tile * dv; i += nthreads) {
                const int key = i / dv, d = i % dv, kp = base + key;
                T val = from_f32<T>(0.f);
                if (kp >= s_lo && kp <= s_hi)
                    val = v_pages[(((size_t)bt[kp / page_size] * Hkv + hk) * page_size + kp % page_size) * dv + d];
                Vs[(size_t)key * dv + d] = val;
            }
        }
        __syncthreads();
        const int c0 = base + wk * 32;                          // this warp's 32 keys
        if (!live || c0 > s_hi || c0 + 31 < s_lo) continue;     // uniform over the warp (barriers are outside)
        const int kp = c0 + lane;
        const bool valid = kp >= s_lo && kp <= s_hi;
        const T* kr = Ks + (size_t)(wk * 32 + lane) * krow;
        const float* qh = qs + wh * dk;
        float dot = 0.f;
        for (int d = 0; d < dk; d += VEC) {
            float kv[8];
            if constexpr (sizeof(T) == 4) {
                const float4 x = *reinterpret_cast<const float4*>(kr + d);
                kv[0] = x.x; kv[1] = x.y; kv[2] = x.z; kv[3] = x.w;
            } else {
                load8(kr + d, kv);
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) dot = fmaf(qh[d + e], kv[e], dot);
        }
        float sc = -INFINITY;
        if (valid) {
            sc = dot * qf;
            if (brow) sc += brow[p - kp];
        }
        const float m_new = fmaxf(m, warp_max(sc));             // at least one key of the chunk is visible
        const float alpha = expf(m - m_new);
        const float pr = valid ? expf(sc - m_new) : 0.f;
        l = l * alpha + warp_sum(pr);
        m = m_new;
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= alpha;
        const T* vt = Vs + (size_t)(wk * 32) * dv;
#pragma unroll 4
        for (int j = 0; j < 32; ++j) {
            const float pj = __shfl_sync(0xffffffffu, pr, j);
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                const int d = lane + 32 * i;
                if (d < dv) acc[i] = fmaf(pj, to_f32(vt[(size_t)j * dv + d]), acc[i]);
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) so[warp * dv + d] = acc[i];
    }
    if (lane == 0) { sml[warp * 2] = m; sml[warp * 2 + 1] = l; }
    __syncthreads();
    // the key sub-tiles of a head meet in sub-tile order
    for (int hh = 0; hh < nh; ++hh) {
        float mm = -INFINITY;
        for (int k = 0; k < KS; ++k)
            if (sml[(k * HG + hh) * 2 + 1] > 0.f) mm = fmaxf(mm, sml[(k * HG + hh) * 2]);
        float ll = 0.f;
        for (int k = 0; k < KS; ++k) {
            const float lw = sml[(k * HG + hh) * 2 + 1];
            if (lw > 0.f) ll += lw * expf(sml[(k * HG + hh) * 2] - mm);
        }
        const size_t pi = ((size_t)t * H + h0 + hh) * nsplit + split;
        for (int d = tid; d < dv; d += nthreads) {
            float o = 0.f;
            for (int k = 0; k < KS; ++k) {
                const float lw = sml[(k * HG + hh) * 2 + 1];
                if (lw > 0.f) o += so[(k * HG + hh) * dv + d] * expf(sml[(k * HG + hh) * 2] - mm);
            }
            part_o[pi * dv + d] = o;
        }
        if (tid == 0) { part_ml[pi * 2] = mm; part_ml[pi * 2 + 1] = ll; }
    }
}

// One warp per (token, head): out = out_scale * sum_s o_s e^(m_s - m) / sum_s l_s e^(m_s - m), in split order.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_bias_merge_kernel(const float* part_o, const float* part_ml, const int* __restrict__ positions,
                            T* __restrict__ out, long long out_stride, int T_tokens, int H, int dv, int nsplit,
                            float out_scale) {
    pdl_wait();
    pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long gw = (long long)blockIdx.x * WARPS + warp;
    if (gw >= (long long)T_tokens * H) return;
    const int t = (int)(gw / H), h = (int)(gw % H);
    const int used = min(nsplit, positions[t] / SPLIT + 1);
    const size_t base = ((size_t)t * H + h) * nsplit;
    float mm = -INFINITY;
    for (int s = 0; s < used; ++s)
        if (part_ml[(base + s) * 2 + 1] > 0.f) mm = fmaxf(mm, part_ml[(base + s) * 2]);
    float ll = 0.f;
    constexpr int NACC = MAX_D / 32;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    for (int s = 0; s < used; ++s) {
        const float ls = part_ml[(base + s) * 2 + 1];
        if (!(ls > 0.f)) continue;
        const float f = expf(part_ml[(base + s) * 2] - mm);
        ll += ls * f;
#pragma unroll
        for (int i = 0; i < NACC; ++i) {
            const int d = lane + 32 * i;
            if (d < dv) acc[i] = fmaf(part_o[(base + s) * dv + d], f, acc[i]);
        }
    }
    T* orow = out + (size_t)t * out_stride + (size_t)h * dv;
    const float inv = out_scale / ll;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) orow[d] = from_f32<T>(acc[i] * inv);
    }
}

// ------------------------------------------------------------------------------------------------ prompt portions
constexpr int BQ = 64, BK = 32, THREADS = 256;

// grid (H, tiles).  A tile is up to 64 consecutive new tokens of one request (request, first flat token, rows).
template <typename T>
__global__ void __launch_bounds__(THREADS)
attention_bias_tiled_kernel(const T* q, long long q_stride, const T* k_pages, const T* v_pages,
                            const int* __restrict__ block_table, int bt_stride, const int* __restrict__ tiles,
                            const int* __restrict__ positions, T* __restrict__ out, long long out_stride, int H, int Hkv,
                            int dk, int dv, int page_size, BiasArgs a) {
    extern __shared__ float sm[];
    const int qrow = dk + 1;
    float* Qs = sm;                         // [BQ][dk+1]   queries times scale times their position's factor
    float* Kt = Qs + BQ * qrow;             // [dk][BK]
    float* Vs = Kt + dk * BK;               // [BK][dv]
    float* Ps = Vs + BK * dv;               // [BQ][BK+1]
    float* Bs = Ps + BQ * (BK + 1);         // [BQ+BK]      the head's bias at the distances this tile pair can have
    pdl_wait();
    pdl_launch();
    const int tile = blockIdx.y, h = blockIdx.x;
    const int seq = tiles[tile * 3], tok0 = tiles[tile * 3 + 1], rows = tiles[tile * 3 + 2];
    const int pos0 = positions[tok0], pos_max = pos0 + rows - 1;
    const int hk = h / (H / Hkv);
    const int* bt = block_table + (size_t)seq * bt_stride;
    const int tid = threadIdx.x, ty = tid >> 3, tx = tid & 7;          // rows 2ty, 2ty+1; keys 4tx..4tx+3; dims tx + 8i
    int first_key = 0;
    if (a.window > 0 && pos0 - a.window + 1 > 0) first_key = pos0 - a.window + 1;
    const float* brow = a.dist_bias ? a.dist_bias + (size_t)h * a.n_dist : nullptr;

    for (int i = tid; i < BQ * dk; i += THREADS) {
        const int r = i / dk, d = i % dk;
        float v = 0.f;
        if (r < rows) {
            const float qf = a.scale * (a.q_scale ? a.q_scale[pos0 + r] : 1.0f);
            v = to_f32(q[(size_t)(tok0 + r) * q_stride + (size_t)h * dk + d]) * qf;
        }
        Qs[r * qrow + d] = v;
    }
    constexpr int MAXI = MAX_D / 8;
    float o[2][MAXI];
#pragma unroll
    for (int i = 0; i < MAXI; ++i) { o[0][i] = 0.f; o[1][i] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int nd = (dv + 7) / 8;
    const int q0 = pos0 + 2 * ty;           // absolute position of this thread's first row
    constexpr int VEC = 16 / sizeof(T);

    for (int j = first_key / BK; j <= pos_max / BK; ++j) {
        __syncthreads();                    // the previous tile is no longer read (and Qs is complete)
        const int kpieces = dk / VEC;
        for (int i = tid; i < BK * kpieces; i += THREADS) {
            const int key = i % BK, piece = i / BK;
            const int kp = j * BK + key;
            float kf[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) kf[e] = 0.f;
            if (kp <= pos_max && kp >= first_key) {
                const int page = bt[kp / page_size];
                const T* src = k_pages + (((size_t)page * Hkv + hk) * page_size + kp % page_size) * dk + piece * VEC;
                if constexpr (sizeof(T) == 4) {
                    const float4 x = *reinterpret_cast<const float4*>(src);
                    kf[0] = x.x; kf[1] = x.y; kf[2] = x.z; kf[3] = x.w;
                } else {
                    load8(src, kf);
                }
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) Kt[(piece * VEC + e) * BK + key] = kf[e];
        }
        for (int i = tid; i < BK * dv; i += THREADS) {
            const int key = i / dv, d = i % dv;
            const int kp = j * BK + key;
            float v = 0.f;
            if (kp <= pos_max && kp >= first_key) {
                const int page = bt[kp / page_size];
                v = to_f32(v_pages[(((size_t)page * Hkv + hk) * page_size + kp % page_size) * dv + d]);
            }
            Vs[key * dv + d] = v;
        }
        // distances between this query tile and this key tile: pos0 - (j*BK + BK-1) .. pos_max - j*BK
        const int dist0 = pos0 - (j * BK + BK - 1);
        if (brow)
            for (int i = tid; i < BQ + BK; i += THREADS) {
                const int dist = dist0 + i;
                Bs[i] = (dist >= 0 && dist < a.n_dist) ? brow[dist] : 0.f;
            }
        __syncthreads();
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        const float* qa = Qs + (2 * ty) * qrow;
        const float* qb = qa + qrow;
        for (int d = 0; d < dk; ++d) {
            const float4 kv = *reinterpret_cast<const float4*>(Kt + d * BK + 4 * tx);
            const float x = qa[d], y = qb[d];
            s[0][0] = fmaf(x, kv.x, s[0][0]); s[0][1] = fmaf(x, kv.y, s[0][1]);
            s[0][2] = fmaf(x, kv.z, s[0][2]); s[0][3] = fmaf(x, kv.w, s[0][3]);
            s[1][0] = fmaf(y, kv.x, s[1][0]); s[1][1] = fmaf(y, kv.y, s[1][1]);
            s[1][2] = fmaf(y, kv.z, s[1][2]); s[1][3] = fmaf(y, kv.w, s[1][3]);
        }
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int qp = q0 + r;
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int kp = j * BK + 4 * tx + c;
                const bool vis = kp <= qp && qp <= pos_max && (a.window <= 0 || kp > qp - a.window);
                float sc = s[r][c];
                if (brow && vis) sc += Bs[qp - kp - dist0];
                s[r][c] = vis ? sc : -INFINITY;
                mx = fmaxf(mx, s[r][c]);
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            const float m_new = fmaxf(m_run[r], mx);
            const float muse = m_new == -INFINITY ? 0.f : m_new;
            alpha[r] = expf(m_run[r] - muse);
            float rs = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float p = expf(s[r][c] - muse);
                Ps[(2 * ty + r) * (BK + 1) + 4 * tx + c] = p;
                rs += p;
            }
            rs += __shfl_xor_sync(0xffffffffu, rs, 1);
            rs += __shfl_xor_sync(0xffffffffu, rs, 2);
            rs += __shfl_xor_sync(0xffffffffu, rs, 4);
            l_run[r] = l_run[r] * alpha[r] + rs;
            m_run[r] = m_new;
        }
        __syncwarp();                       // a row's 8 threads are lanes of one warp: its p values are in place
#pragma unroll
        for (int i = 0; i < MAXI; ++i) {
            if (i < nd) { o[0][i] *= alpha[0]; o[1][i] *= alpha[1]; }
        }
        const float* pa = Ps + (2 * ty) * (BK + 1);
        const float* pb = pa + (BK + 1);
        for (int key = 0; key < BK; ++key) {
            const float p0 = pa[key], p1 = pb[key];
            const float* vr = Vs + key * dv + tx;
#pragma unroll
            for (int i = 0; i < MAXI; ++i) {
                if (i < nd && tx + 8 * i < dv) {
                    const float v = vr[8 * i];
                    o[0][i] = fmaf(p0, v, o[0][i]);
                    o[1][i] = fmaf(p1, v, o[1][i]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = 2 * ty + r;
        if (row >= rows) continue;
        const float inv = a.out_scale / l_run[r];
        T* orow = out + (size_t)(tok0 + row) * out_stride + (size_t)h * dv;
#pragma unroll
        for (int i = 0; i < MAXI; ++i)
            if (i < nd && tx + 8 * i < dv) orow[tx + 8 * i] = from_f32<T>(o[r][i] * inv);
    }
}

int check_sizes(int H, int Hkv, int dk, int dv, int page_size, int dtype) {
    const int vec = dtype == MLLM_F32 ? 4 : 8;
    if (dtype != MLLM_F32 && dtype != MLLM_BF16) return mllm_fail(1, "attention_bias: unknown dtype code %d", dtype);
    if (dk <= 0 || dk % 8 != 0 || dk > MAX_D)
        return mllm_fail(1, "attention_bias: key size %d is not a multiple of 8 in 8..%d", dk, MAX_D);
    if (dv <= 0 || dv > MAX_D) return mllm_fail(1, "attention_bias: value size %d is not in 1..%d", dv, MAX_D);
    (void)vec;
    if (Hkv <= 0 || H % Hkv != 0) return mllm_fail(1, "attention_bias: %d heads over %d key/value heads", H, Hkv);
    if (page_size <= 0) return mllm_fail(1, "attention_bias: page size %d", page_size);
    return 0;
}

}  // namespace

MLLM_EXPORT int mllm_attention_bias_split_keys() { return SPLIT; }

// impl: 0 simt, 1 tiled (needs tiles), 2 split (single tokens; needs part_o [T*H*nsplit*dv], part_ml [T*H*nsplit*2]).
MLLM_EXPORT int mllm_attention_bias(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                    const int* block_table, int bt_stride, const int* token_seq, const int* positions,
                                    const int* tiles, int n_tiles, void* out, long long out_stride, float* part_o,
                                    float* part_ml, int nsplit, int T, int H, int Hkv, int dk, int dv, int page_size,
                                    float scale, float out_scale, const float* dist_bias, int n_dist,
                                    const float* q_scale, int window, int dtype, int impl, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (int rc = check_sizes(H, Hkv, dk, dv, page_size, dtype)) return rc;
    BiasArgs a{dist_bias, n_dist, q_scale, scale, out_scale, window};
    const long long warps = (long long)T * H;
    const long long blocks = (warps + WARPS - 1) / WARPS;
    if (blocks > 2147483647LL) return mllm_fail(1, "attention_bias: too many (token, head) pairs");
    using bf = __nv_bfloat16;
    if (impl == 0) {
        if (dtype == MLLM_F32)
            MLLM_CUDA(mllm_launch(attention_bias_simt_kernel<float>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream,
                                  true, (const float*)q, q_stride, (const float*)k_pages, (const float*)v_pages,
                                  block_table, bt_stride, token_seq, positions, (float*)out, out_stride, T, H, Hkv, dk, dv,
                                  page_size, a));
        else
            MLLM_CUDA(mllm_launch(attention_bias_simt_kernel<bf>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream, true,
                                  (const bf*)q, q_stride, (const bf*)k_pages, (const bf*)v_pages, block_table, bt_stride,
                                  token_seq, positions, (bf*)out, out_stride, T, H, Hkv, dk, dv, page_size, a));
        return 0;
    }
    if (impl == 1) {
        if (!tiles || n_tiles <= 0) return mllm_fail(1, "attention_bias: the tiled kernel needs the step's tile list");
        const size_t smem = sizeof(float) * ((size_t)BQ * (dk + 1) + (size_t)dk * BK + (size_t)BK * dv + BQ * (BK + 1) + BQ + BK);
        if (smem > 227 * 1024) return mllm_fail(1, "attention_bias: sizes %d / %d need %zu bytes of shared memory", dk, dv, smem);
        if (dtype == MLLM_F32) {
            MLLM_CUDA(cudaFuncSetAttribute(attention_bias_tiled_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            MLLM_CUDA(mllm_launch(attention_bias_tiled_kernel<float>, dim3(H, n_tiles), dim3(THREADS), smem, stream, true,
                                  (const float*)q, q_stride, (const float*)k_pages, (const float*)v_pages, block_table,
                                  bt_stride, tiles, positions, (float*)out, out_stride, H, Hkv, dk, dv, page_size, a));
        } else {
            MLLM_CUDA(cudaFuncSetAttribute(attention_bias_tiled_kernel<bf>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            MLLM_CUDA(mllm_launch(attention_bias_tiled_kernel<bf>, dim3(H, n_tiles), dim3(THREADS), smem, stream, true,
                                  (const bf*)q, q_stride, (const bf*)k_pages, (const bf*)v_pages, block_table, bt_stride,
                                  tiles, positions, (bf*)out, out_stride, H, Hkv, dk, dv, page_size, a));
        }
        return 0;
    }
    if (impl == 2) {
        if (!part_o || !part_ml || nsplit <= 0) return mllm_fail(1, "attention_bias: the split kernel needs scratch for its partial results");
        const int R = H / Hkv;
        int HG = R >= 4 ? 4 : (R >= 2 ? 2 : 1), KS = 4 / HG;
        const size_t es = dtype == MLLM_F32 ? 4 : 2, vec = 16 / es;
        auto bytes = [&](int ks) {
            const size_t tile = 32 * (size_t)ks;
            return tile * (dk + vec) * es + ((tile * dv + vec - 1) / vec) * vec * es + sizeof(float) * ((size_t)HG * dk + 4 * (size_t)dv + 8);
        };
        while (KS > 1 && bytes(KS) > 96 * 1024) KS /= 2;
        const size_t smem = bytes(KS);
        const int chunks = (R + HG - 1) / HG;
        if ((long long)Hkv * chunks > 65535 || T > 65535) return mllm_fail(1, "attention_bias: %d heads x %d tokens exceed the split kernel's grid", H, T);
        const dim3 grid(nsplit, Hkv * chunks, T), block(32 * HG * KS);
        if (dtype == MLLM_F32) {
            if (smem > 48 * 1024) MLLM_CUDA(cudaFuncSetAttribute(attention_bias_split_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            MLLM_CUDA(mllm_launch(attention_bias_split_kernel<float>, grid, block, smem, stream, true,
                                  (const float*)q, q_stride, (const float*)k_pages, (const float*)v_pages, block_table,
                                  bt_stride, token_seq, positions, part_o, part_ml, H, Hkv, dk, dv, page_size, HG, KS, a));
            MLLM_CUDA(mllm_launch(attention_bias_merge_kernel<float>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream, true,
                                  (const float*)part_o, (const float*)part_ml, positions, (float*)out, out_stride, T, H, dv,
                                  nsplit, out_scale));
        } else {
            if (smem > 48 * 1024) MLLM_CUDA(cudaFuncSetAttribute(attention_bias_split_kernel<bf>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            MLLM_CUDA(mllm_launch(attention_bias_split_kernel<bf>, grid, block, smem, stream, true,
                                  (const bf*)q, q_stride, (const bf*)k_pages, (const bf*)v_pages, block_table, bt_stride,
                                  token_seq, positions, part_o, part_ml, H, Hkv, dk, dv, page_size, HG, KS, a));
            MLLM_CUDA(mllm_launch(attention_bias_merge_kernel<bf>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream, true,
                                  (const float*)part_o, (const float*)part_ml, positions, (bf*)out, out_stride, T, H, dv,
                                  nsplit, out_scale));
        }
        return 0;
    }
    return mllm_fail(1, "attention_bias: unknown implementation %d", impl);
}

// rows of src [T, heads * d] (row stride given) to their page slots in pages [num_pages, heads, page_size, d]
namespace {
template <typename T>
__global__ void __launch_bounds__(256)
paged_write_kernel(const T* src, long long row_stride, T* __restrict__ pages, const int* __restrict__ slots, int T_tokens,
                   int heads, int d, int page_size) {
    pdl_wait();
    pdl_launch();
    const int per = heads * d;
    const long long total = (long long)T_tokens * per;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / per), c = (int)(i % per);
        const int slot = slots[t];
        if (slot < 0) continue;
        const int h = c / d, e = c % d;
        pages[(((size_t)(slot / page_size) * heads + h) * page_size + slot % page_size) * d + e] = src[(size_t)t * row_stride + c];
    }
}
}  // namespace

// keys [T, heads * dk] and values [T, heads * dv] of the step to their page slots in one launch
namespace {
template <typename T>
__global__ void __launch_bounds__(256)
paged_write_kv_kernel(const T* k, long long k_stride, const T* v, long long v_stride, T* __restrict__ k_pages,
                      T* __restrict__ v_pages, const int* __restrict__ slots, int T_tokens, int heads, int dk, int dv,
                      int page_size) {
    pdl_wait();
    pdl_launch();
    const int pk = heads * dk, per = heads * (dk + dv);
    const long long total = (long long)T_tokens * per;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / per), c = (int)(i % per);
        const int slot = slots[t];
        if (slot < 0) continue;
        const size_t row = (size_t)(slot / page_size) * heads;
        const int off = slot % page_size;
        if (c < pk) {
            const int h = c / dk, e = c % dk;
            k_pages[((row + h) * page_size + off) * dk + e] = k[(size_t)t * k_stride + c];
        } else {
            const int cc = c - pk, h = cc / dv, e = cc % dv;
            v_pages[((row + h) * page_size + off) * dv + e] = v[(size_t)t * v_stride + cc];
        }
    }
}
}  // namespace

MLLM_EXPORT int mllm_paged_write_kv(const void* k, long long k_stride, const void* v, long long v_stride, void* k_pages,
                                    void* v_pages, const int* slots, int T, int heads, int dk, int dv, int page_size,
                                    int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    const long long total = (long long)T * heads * (dk + dv);
    const int grid = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
    if (dtype == MLLM_F32)
        MLLM_CUDA(mllm_launch(paged_write_kv_kernel<float>, dim3(grid), dim3(256), 0, stream, true, (const float*)k, k_stride,
                              (const float*)v, v_stride, (float*)k_pages, (float*)v_pages, slots, T, heads, dk, dv, page_size));
    else if (dtype == MLLM_BF16)
        MLLM_CUDA(mllm_launch(paged_write_kv_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, true,
                              (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride, (__nv_bfloat16*)k_pages,
                              (__nv_bfloat16*)v_pages, slots, T, heads, dk, dv, page_size));
    else
        return mllm_fail(1, "paged_write_kv: unknown dtype code %d", dtype);
    return 0;
}

MLLM_EXPORT int mllm_paged_write(const void* src, long long row_stride, void* pages, const int* slots, int T, int heads,
                                 int d, int page_size, int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    const long long total = (long long)T * heads * d;
    const int grid = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
    if (dtype == MLLM_F32)
        MLLM_CUDA(mllm_launch(paged_write_kernel<float>, dim3(grid), dim3(256), 0, stream, true, (const float*)src, row_stride,
                              (float*)pages, slots, T, heads, d, page_size));
    else if (dtype == MLLM_BF16)
        MLLM_CUDA(mllm_launch(paged_write_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, true,
                              (const __nv_bfloat16*)src, row_stride, (__nv_bfloat16*)pages, slots, T, heads, d, page_size));
    else
        return mllm_fail(1, "paged_write: unknown dtype code %d", dtype);
    return 0;
}
