// Attention over a cache of latents: every token keeps ONE row [c (R) | k_rot (dr) | padding], shared by all heads.
// A head's unrotated key is W_uk c and its value W_uv c, so with qa = W_uk^T q_unrotated the score is
// (qa . c + q_rot . k_rot) * scale and the head's output is W_uv (sum_j p_j c_j): attention runs in the latent space
// (one key/value head of R + dr key columns whose first R columns are also the value), and the two per-head products
// are small matrix products before and after it.
//
//   latent_prepare   per token: RMS norm of the latent (32-bit) -> cache row; rotation of the shared key part and of
//                    every head's rotated query part at the token's position (angles, cos and sin 32-bit) -> cache row
//                    and columns R.. of qa.
//   headwise_linear  out[t][h][n] = sum_k in[t][h][k] W[h][n][k] (optionally times sigmoid(gate[t][h][n])):
//                    the absorbed query (W = W_uk^T per head) and the head outputs (W = W_uv per head, with the gate).
//                    Three kernels: CUDA-core tiles (32-bit weights, odd sizes), tensor-core tiles (bfloat16 weights,
//                    more than 16 tokens), and for up to 16 tokens a CTA per (token, head) that streams its weights.
//   latent_attention one CTA per (split of `span` keys, token, block of 8 heads): key rows are staged once for all the
//                    heads of the block in chunks of 32 that start at multiples of 32 from position 0; a warp is a
//                    head, its lanes are the 32 keys for the scores and 64 latent columns at a time for the weighted
//                    sum; online softmax in 32-bit with expf.  Partial (o, m, l) per split, merged in split order by
//                    latent_merge.  Splits and chunks are fixed ranges of positions, so at one span a token's sums run
//                    in the same order whether it came in a prompt portion, alone, or in a batch (the caller takes
//                    short splits for steps of single tokens, to fill the GPU, and long ones otherwise).
#include "common.cuh"

namespace {

constexpr int HB = 8;           // heads (warps) per CTA
constexpr int MAX_SMEM = 227 * 1024;    // dynamic shared memory a CTA can have on this GPU
constexpr int MAX_R = 512;      // largest latent size
constexpr int MAX_DK = 1024;    // largest R + dr

template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* proj, long long ld, int q_off, int dkv_off, int H, int dn, int dr, int R, int rot_dims,
                      const int* positions, const int* slot_mapping, const float* __restrict__ freq, float mscale,
                      const float* __restrict__ normw, float eps, T* pages, int row, float* qa, int write) {
    __shared__ float scratch[33];
    pdl_wait();
    const int t = blockIdx.x;
    const float p = (float)positions[t];
    const T* x = proj + (size_t)t * ld;
    const int half = rot_dims / 2;
    if (dkv_off >= 0 && write) {
        const T* d = x + dkv_off;
        T* dst = pages + (size_t)slot_mapping[t] * row;
        float ss = 0.f;
        for (int i = threadIdx.x; i < R; i += blockDim.x) {
            const float v = to_f32(d[i]);
            ss = fmaf(v, v, ss);
        }
        const float r = sqrtf(block_sum(ss, scratch) / (float)R + eps);
        for (int i = threadIdx.x; i < R; i += blockDim.x) dst[i] = from_f32<T>(to_f32(d[i]) / r * normw[i]);
        for (int i = threadIdx.x; i < dr; i += blockDim.x) {
            float o;
            if (i < rot_dims) {
                const int k = i < half ? i : i - half;
                float sn, cs;
                sincosf(p * freq[k], &sn, &cs);
                sn *= mscale;
                cs *= mscale;
                const float u = to_f32(d[R + k]), v = to_f32(d[R + half + k]);
                o = i < half ? u * cs - v * sn : v * cs + u * sn;
            } else {
                o = to_f32(d[R + i]);
            }
            dst[R + i] = from_f32<T>(o);
        }
    }
    const int dq = dn + dr, dk = R + dr;
    for (int j = threadIdx.x; j < H * dr; j += blockDim.x) {
        const int h = j / dr, i = j % dr;
        const T* q = x + q_off + (size_t)h * dq + dn;
        float o;
        if (i < rot_dims) {
            const int k = i < half ? i : i - half;
            float sn, cs;
            sincosf(p * freq[k], &sn, &cs);
            sn *= mscale;
            cs *= mscale;
            const float u = to_f32(q[k]), v = to_f32(q[half + k]);
            o = i < half ? u * cs - v * sn : v * cs + u * sn;
        } else {
            o = to_f32(q[i]);
        }
        qa[((size_t)t * H + h) * dk + R + i] = o;
    }
}

// out[t][h][n] = sum_k in[t][h][k] * W[h][n][k]  (* sigmoid(gate[t][h * N + n])).  32 tokens x 64 columns per CTA and head.
template <typename TI, typename TW, typename TO>
__global__ void __launch_bounds__(256)
headwise_linear_kernel(const TI* in, long long ld_in, int in_head, const TW* __restrict__ W, TO* out, long long ld_out,
                       int out_head, const TO* gate, long long ld_gate, int Tn, int N, int K) {
    __shared__ float As[32][33];
    __shared__ float Ws[64][33];
    pdl_wait();
    const int h = blockIdx.z, t0 = blockIdx.x * 32, n0 = blockIdx.y * 64;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const TW* Wh = W + (size_t)h * N * K;
    float acc[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += 32) {
        for (int i = threadIdx.x; i < 32 * 32; i += 256) {
            const int r = i >> 5, c = i & 31;
            As[r][c] = (t0 + r < Tn && k0 + c < K) ? to_f32(in[(size_t)(t0 + r) * ld_in + (size_t)h * in_head + k0 + c]) : 0.f;
        }
        for (int i = threadIdx.x; i < 64 * 32; i += 256) {
            const int r = i >> 5, c = i & 31;
            Ws[r][c] = (n0 + r < N && k0 + c < K) ? to_f32(Wh[(size_t)(n0 + r) * K + k0 + c]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < 32; ++kk) {
            const float a0 = As[ty * 2][kk], a1 = As[ty * 2 + 1][kk];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float w = Ws[tx + 16 * i][kk];
                acc[0][i] = fmaf(a0, w, acc[0][i]);
                acc[1][i] = fmaf(a1, w, acc[1][i]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int t = t0 + ty * 2 + j;
        if (t >= Tn) continue;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int n = n0 + tx + 16 * i;
            if (n >= N) continue;
            float v = acc[j][i];
            if (gate) v *= 1.0f / (1.0f + expf(-to_f32(gate[(size_t)t * ld_gate + (size_t)h * N + n])));
            out[(size_t)t * ld_out + (size_t)h * out_head + n] = from_f32<TO>(v);
        }
    }
}

// The same products for few tokens (decode steps): grid (tokens, heads, column blocks of 64), 8 warps.  The token's K
// inputs of the head are staged in shared memory as 32-bit; a warp owns 8 columns, its lanes split K (the 8 weight rows'
// loads in flight together), the sums meet by a butterfly.
template <typename TI, typename TW, typename TO>
__global__ void __launch_bounds__(256)
headwise_rows_kernel(const TI* in, long long ld_in, int in_head, const TW* __restrict__ W, TO* out, long long ld_out,
                     int out_head, const TO* gate, long long ld_gate, int N, int K) {
    extern __shared__ float hx[];                                // [K]
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y;
    const TI* x = in + (size_t)t * ld_in + (size_t)h * in_head;
    for (int k = threadIdx.x; k < K; k += 256) hx[k] = to_f32(x[k]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.z * 64 + warp * 8;
    if (n0 >= N) return;
    const TW* Wh = W + (size_t)h * N * K;
    float acc[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) acc[u] = 0.f;
    for (int k = lane; k < K; k += 32) {
        const float xv = hx[k];
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[u] = fmaf(xv, to_f32(Wh[(size_t)min(n0 + u, N - 1) * K + k]), acc[u]);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        float v = warp_sum(acc[u]);
        const int n = n0 + u;
        if (lane == 0 && n < N) {
            if (gate) v *= 1.0f / (1.0f + expf(-to_f32(gate[(size_t)t * ld_gate + (size_t)h * N + n])));
            out[(size_t)t * ld_out + (size_t)h * out_head + n] = from_f32<TO>(v);
        }
    }
}

// grid (splits, tokens, head blocks); dynamic shared memory: HB * dkp floats of queries, then two chunks of 32 key rows
// of `kw` 32-bit words each (kw = a row's words + 4: rows stay 16-byte aligned for cp.async and 128-bit reads, and eight
// lanes reading 16 bytes of eight consecutive rows touch all 32 banks).  A CTA walks the keys [split * span, ...) of its
// token in chunks of 32, the next chunk's rows in flight (cp.async) while the current one is used.
__device__ __forceinline__ void cp16(void* dst, const void* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

template <typename T, int NACC>
__global__ void __launch_bounds__(HB * 32)
latent_attention_kernel(const float* qa, const T* pages, int row, const int* block_table, int bt_stride,
                        const int* token_seq, const int* positions, float* part_o, float* part_ml, int nsplit, int H,
                        int R, int dk, int ps, float scale, int kw, int span) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int EPW = 4 / sizeof(T);                  // elements per 32-bit word
    constexpr int V = 16 / sizeof(T);                   // elements per 16 bytes
    const int dkp = (dk + V - 1) / V * V;               // the padding of a cache row is zero: whole 16-byte pieces are used
    float* qs = reinterpret_cast<float*>(smem_raw);
    uint32_t* ks = reinterpret_cast<uint32_t*>(qs + HB * dkp);
    pdl_wait();
    const int t = blockIdx.y, split = blockIdx.x;
    const int p = positions[t];
    const int k_lo = split * span;
    if (k_lo > p) return;
    const int k_hi = min(k_lo + span - 1, p);           // inclusive
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h0 = blockIdx.z * HB, h = h0 + warp;
    const int nh = min(HB, H - h0);
    const int* bt = block_table + (size_t)token_seq[t] * bt_stride;
    const int vec_per_row = row / V;                    // rows are padded to multiples of 16 bytes
    auto stage = [&](int base, int buf) {
        const int nk = min(32, k_hi - base + 1);
        uint32_t* dst = ks + buf * 32 * kw;
        for (int i = threadIdx.x; i < nk * vec_per_row; i += HB * 32) {
            const int j = i / vec_per_row, v = i - j * vec_per_row;
            const int pos = base + j;
            const T* src = pages + ((size_t)bt[pos / ps] * ps + pos % ps) * row;
            cp16(dst + j * kw + v * 4, reinterpret_cast<const unsigned char*>(src) + 16 * v);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(k_lo, 0);
    for (int i = threadIdx.x; i < nh * dkp; i += blockDim.x) {
        const int hh = i / dkp, d = i - hh * dkp;
        qs[i] = d < dk ? qa[((size_t)t * H + h0 + hh) * dk + d] : 0.f;
    }
    float m = -INFINITY, l = 0.f, acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    const float* q = qs + warp * dkp;
    int buf = 0;
    for (int base = k_lo; base <= k_hi; base += 32, buf ^= 1) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();            // this chunk (and the queries) are in; the other buffer has been used
        if (base + 32 <= k_hi) stage(base + 32, buf ^ 1);
        const int nk = min(32, k_hi - base + 1);
        if (h >= H) continue;
        const uint32_t* kc = ks + buf * 32 * kw;
        float s = -INFINITY;
        if (lane < nk) {
            const uint32_t* kr = kc + lane * kw;
            float d0 = 0.f, d1 = 0.f;
            for (int d = 0; d < dkp; d += V) {
                const uint4 kv = *reinterpret_cast<const uint4*>(kr + d / EPW);
                const float4 qa0 = *reinterpret_cast<const float4*>(q + d);
                if constexpr (sizeof(T) == 4) {
                    d0 = fmaf(qa0.x, __uint_as_float(kv.x), d0);
                    d1 = fmaf(qa0.y, __uint_as_float(kv.y), d1);
                    d0 = fmaf(qa0.z, __uint_as_float(kv.z), d0);
                    d1 = fmaf(qa0.w, __uint_as_float(kv.w), d1);
                } else {
                    const float4 qa1 = *reinterpret_cast<const float4*>(q + d + 4);
                    d0 = fmaf(qa0.x, __uint_as_float(kv.x << 16), d0);
                    d1 = fmaf(qa0.y, __uint_as_float(kv.x & 0xffff0000u), d1);
                    d0 = fmaf(qa0.z, __uint_as_float(kv.y << 16), d0);
                    d1 = fmaf(qa0.w, __uint_as_float(kv.y & 0xffff0000u), d1);
                    d0 = fmaf(qa1.x, __uint_as_float(kv.z << 16), d0);
                    d1 = fmaf(qa1.y, __uint_as_float(kv.z & 0xffff0000u), d1);
                    d0 = fmaf(qa1.z, __uint_as_float(kv.w << 16), d0);
                    d1 = fmaf(qa1.w, __uint_as_float(kv.w & 0xffff0000u), d1);
                }
            }
            s = (d0 + d1) * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float alpha = expf(m - m_new);           // 0 at the first chunk (m = -inf)
        const float pj = lane < nk ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(pj);
        m = m_new;
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= alpha;
        // the weighted sum: a lane owns the column pairs (2 * lane, 2 * lane + 1) + 64 * i
        for (int j = 0; j < nk; ++j) {
            const float w = __shfl_sync(0xffffffffu, pj, j);
            const uint32_t* kr = kc + j * kw;
#pragma unroll
            for (int i = 0; i < NACC / 2; ++i) {
                const int d = 2 * lane + 64 * i;
                if (d < R) {
                    float c0, c1;
                    if constexpr (sizeof(T) == 4) {
                        const float2 c = *reinterpret_cast<const float2*>(kr + d);
                        c0 = c.x; c1 = c.y;
                    } else {
                        const uint32_t c = kr[d >> 1];
                        c0 = __uint_as_float(c << 16); c1 = __uint_as_float(c & 0xffff0000u);
                    }
                    acc[2 * i] = fmaf(w, c0, acc[2 * i]);
                    acc[2 * i + 1] = fmaf(w, c1, acc[2 * i + 1]);
                }
            }
        }
    }
    if (h >= H) return;
    const size_t o = ((size_t)t * H + h) * nsplit + split;
#pragma unroll
    for (int i = 0; i < NACC / 2; ++i) {
        const int d = 2 * lane + 64 * i;
        if (d < R) part_o[o * R + d] = acc[2 * i];
        if (d + 1 < R) part_o[o * R + d + 1] = acc[2 * i + 1];
    }
    if (lane == 0) {
        part_ml[o * 2] = m;
        part_ml[o * 2 + 1] = l;
    }
}

// One warp per (token, head): out = sum_s o_s e^(m_s - M) / sum_s l_s e^(m_s - M) over the splits the token has.
__global__ void __launch_bounds__(256)
latent_merge_kernel(const float* part_o, const float* part_ml, const int* positions, float* out, int nsplit, int TH, int H,
                    int R, int span) {
    pdl_wait();
    const int th = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (th >= TH) return;
    const int ns = positions[th / H] / span + 1;
    const size_t o = (size_t)th * nsplit;
    float M = -INFINITY;
    for (int s = 0; s < ns; ++s) M = fmaxf(M, part_ml[(o + s) * 2]);
    float L = 0.f;
    for (int s = 0; s < ns; ++s) L += part_ml[(o + s) * 2 + 1] * expf(part_ml[(o + s) * 2] - M);
    for (int d = lane; d < R; d += 32) {
        float a = 0.f;
        for (int s = 0; s < ns; ++s) a = fmaf(part_o[(o + s) * R + d], expf(part_ml[(o + s) * 2] - M), a);
        out[(size_t)th * R + d] = a / L;
    }
}

template <typename T, int NACC>
int launch_attention(const float* qa, const void* pages, int row, const int* bt, int bt_stride, const int* token_seq,
                     const int* positions, float* part_o, float* part_ml, int nsplit, int Tn, int H, int R, int dk,
                     int ps, float scale, int span, cudaStream_t stream) {
    const int kw = row * (int)sizeof(T) / 4 + 4;
    const int V = 16 / (int)sizeof(T), dkp = (dk + V - 1) / V * V;
    const size_t smem = (size_t)HB * dkp * 4 + (size_t)2 * 32 * kw * 4;
    static bool raised = false;                     // once per instantiation
    if (smem > 48 * 1024 && !raised) {
        MLLM_CUDA(cudaFuncSetAttribute(latent_attention_kernel<T, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, MAX_SMEM));
        raised = true;
    }
    if (smem > MAX_SMEM) return mllm_fail(1, "latent_attention: rows of %d need %zu bytes of shared memory", dk, smem);
    MLLM_CUDA(mllm_launch(latent_attention_kernel<T, NACC>, dim3(nsplit, Tn, (H + HB - 1) / HB), dim3(HB * 32), smem, stream,
                          true, qa, (const T*)pages, row, bt, bt_stride, token_seq, positions, part_o, part_ml, nsplit, H,
                          R, dk, ps, scale, kw, span));
    return 0;
}

template <typename T>
int pick_attention(int R, const float* qa, const void* pages, int row, const int* bt, int bt_stride, const int* token_seq,
                   const int* positions, float* part_o, float* part_ml, int nsplit, int Tn, int H, int dk, int ps,
                   float scale, int span, cudaStream_t stream) {
    if (R <= 128)
        return launch_attention<T, 4>(qa, pages, row, bt, bt_stride, token_seq, positions, part_o, part_ml, nsplit, Tn, H, R,
                                      dk, ps, scale, span, stream);
    if (R <= 256)
        return launch_attention<T, 8>(qa, pages, row, bt, bt_stride, token_seq, positions, part_o, part_ml, nsplit, Tn, H, R,
                                      dk, ps, scale, span, stream);
    return launch_attention<T, 16>(qa, pages, row, bt, bt_stride, token_seq, positions, part_o, part_ml, nsplit, Tn, H, R, dk,
                                   ps, scale, span, stream);
}


// ------------------------------------------------------------------------------------------------ prompt portions, bfloat16
// The same attention on tensor cores (mma.sync m16n8k16, bfloat16 operands, 32-bit accumulators) for a bfloat16 cache.
// A CTA takes one tile of up to 64 new tokens of one request and one head; warp (rg, cs) owns the 16 query rows rg*16..
// and the latent columns cs*NO*8.. of the result (CW column parts: a warp's output sums stay in registers also for
// latents of 512; the two warps of a row group then split the tile's keys for the scores and share the weights).  Key tile j covers the positions [32j, 32j + 32): its rows come into shared memory by cp.async as
// they lie in the pages (rows nobody sees are zero-filled), the next tile's while the current one is used, and serve
// twice: as keys (all R + dr columns) and, read transposed, as values (the first R columns).  The absorbed queries are
// taken as hi + lo, two bfloat16 terms (hi alone where shared memory cannot hold both: rows beyond 568 columns), so the
// scores keep about 16 bits of them; scores, mask and the online softmax are 32-bit (scores in units of ln 2, ex2.approx); the
// weights enter the second product as p = hi + lo, two bfloat16 terms, so they keep about 16 bits; output sums 32-bit.
constexpr int MQ = 64, MK = 32;
constexpr int PLD = MK + 8;                                      // row stride of the shared weights
constexpr int PAIR_BYTES = 4 * 2 * 16 * PLD * 2 + 4 * 2 * 16 * 4;   // shared weights and maxima of the four row groups
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void ldsm_x4(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x2(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, const uint32_t* b) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = valid ? 16 : 0;                                // 0 bytes read: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float x, float y) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float ex2(float x) {                   // 2^x in one instruction; 2^(-inf) = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// barrier of the two warps (64 threads) of row group rg
__device__ __forceinline__ void pair_sync(int rg) { asm volatile("bar.sync %0, 64;" ::"r"(rg + 1) : "memory"); }

template <int NO, int CW, int QL>
__global__ void __launch_bounds__(128 * CW)
latent_mma_kernel(const float* qa, const __nv_bfloat16* pages, int row, const int* __restrict__ block_table, int bt_stride,
                  const int* __restrict__ tiles, const int* __restrict__ positions, float* out, int H, int R, int dk, int ps,
                  float scale) {
    using bf = __nv_bfloat16;
    extern __shared__ __align__(16) unsigned char smraw[];
    const int srow = dk + 8;                                     // 16 bytes of padding: ldmatrix rows fall on different banks
    bf* Qs = reinterpret_cast<bf*>(smraw);                       // [MQ][dk + 8], and with QL once more for the low terms
    bf* Ql = Qs + MQ * srow;
    bf* Ks = Qs + (QL ? 2 : 1) * MQ * srow;                      // [2][MK][dk + 8]
    bf* Ps = Ks + 2 * MK * srow;                                 // with two column parts: [4 row groups][hi, lo][16][PLD] weights
    float* Mx = reinterpret_cast<float*>(Ps + 4 * 2 * 16 * PLD); // and [4][2][16] row maxima (row sums at the end)
    pdl_wait();
    const int tile = blockIdx.y, h = blockIdx.x;
    const int seq = tiles[tile * 3], tok0 = tiles[tile * 3 + 1], rows = tiles[tile * 3 + 2];
    const int pos0 = positions[tok0], pos_max = pos0 + rows - 1;
    const int* bt = block_table + (size_t)seq * bt_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rg = warp & 3, cs = warp >> 2;
    const int kp8 = dk / 8;
    auto stage = [&](int j, int buf) {                           // key tile j into buffer buf
        bf* kd = Ks + buf * MK * srow;
        for (int i = tid; i < MK * kp8; i += 128 * CW) {
            const int key = i / kp8, piece = i - key * kp8, kp = j * MK + key;
            const bool ok = kp <= pos_max;
            const bf* src = ok ? pages + ((size_t)bt[kp / ps] * ps + kp % ps) * row + piece * 8 : pages;
            cp_async16(kd + key * srow + piece * 8, src, ok);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(0, 0);
    const int dk2 = dk / 2;
    for (int i = tid; i < MQ * dk2; i += 128 * CW) {             // queries as hi (+ lo) bfloat16 terms; rows beyond the tile are zero
        const int r = i / dk2, c = i - r * dk2;
        float2 v = make_float2(0.f, 0.f);
        if (r < rows) v = *reinterpret_cast<const float2*>(qa + ((size_t)(tok0 + r) * H + h) * dk + 2 * c);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(v.x, v.y);
        *reinterpret_cast<__nv_bfloat162*>(Qs + r * srow + 2 * c) = hi;
        if (QL) *reinterpret_cast<__nv_bfloat162*>(Ql + r * srow + 2 * c) = __floats2bfloat162_rn(v.x - __low2float(hi), v.y - __high2float(hi));
    }
    const int r0 = rg * 16 + (lane >> 2);                        // this thread's rows: r0 and r0 + 8 of the tile
    const int qp0 = pos0 + r0, qp1 = qp0 + 8;
    const float sf = scale * LOG2E;
    float o[NO][4];
#pragma unroll
    for (int i = 0; i < NO; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int nct = R / 8 - cs * NO;                             // column tiles of 8 this warp has (may exceed NO or be <= 0)
    const int j_last = pos_max / MK;
    for (int j = 0; j <= j_last; ++j) {
        const int buf = j & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                         // tile j (and the queries) are in; the other buffer is free
        if (j < j_last) stage(j + 1, buf ^ 1);
        const bf* kt = Ks + buf * MK * srow;
        if (j * MK > pos0 + rg * 16 + 15 || rg * 16 >= rows) continue;      // nothing of the tile is seen by this warp's rows
        // With two column parts a row group's two warps share the scores: each multiplies its 16 keys of the tile, the
        // maxima and the weights (hi and lo terms) meet in shared memory on a barrier of the pair's 64 threads.
        constexpr int NS = CW == 2 ? 2 : 4;                      // score tiles of 8 keys per warp
        const int nb = CW == 2 ? cs * 2 : 0;                     // the first of them
        float s[NS][4];
#pragma unroll
        for (int n = 0; n < NS; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
        for (int k0 = 0; k0 < dk; k0 += 16) {
            uint32_t af[4], al[4];
            ldsm_x4(af, Qs + (rg * 16 + (lane & 15)) * srow + k0 + (lane >> 4) * 8);
            if (QL) ldsm_x4(al, Ql + (rg * 16 + (lane & 15)) * srow + k0 + (lane >> 4) * 8);
#pragma unroll
            for (int n = 0; n < NS; ++n) {
                uint32_t bfr[2];
                ldsm_x2(bfr, kt + ((nb + n) * 8 + (lane & 7)) * srow + k0 + ((lane >> 3) & 1) * 8);
                mma_bf16(s[n], af, bfr);
                if (QL) mma_bf16(s[n], al, bfr);
            }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < NS; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kp = j * MK + (nb + n) * 8 + 2 * (lane & 3) + (e & 1);
                const int qp = (e < 2) ? qp0 : qp1;
                const float sc = (kp <= qp && qp <= pos_max) ? s[n][e] * sf : -INFINITY;
                s[n][e] = sc;
                if (e < 2) mx0 = fmaxf(mx0, sc); else mx1 = fmaxf(mx1, sc);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        if constexpr (CW == 2) {
            float* mine = Mx + (rg * 2 + cs) * 16;
            if ((lane & 3) == 0) { mine[lane >> 2] = mx0; mine[8 + (lane >> 2)] = mx1; }
            pair_sync(rg);
            const float* other = Mx + (rg * 2 + (cs ^ 1)) * 16;
            mx0 = fmaxf(mx0, other[lane >> 2]);
            mx1 = fmaxf(mx1, other[8 + (lane >> 2)]);
        }
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
        const float al0 = ex2(m0 - mu0), al1 = ex2(m1 - mu1);
        m0 = mn0; m1 = mn1;
        float rs0 = 0.f, rs1 = 0.f;
        uint32_t phi[2][4], plo[2][4];                           // A fragments of p for the two 16-key steps
        bf* ph = Ps + (rg * 2) * 16 * PLD;                       // the row group's weights: hi terms, then lo terms
        bf* pl = ph + 16 * PLD;
#pragma unroll
        for (int n = 0; n < NS; ++n) {
            const float p0 = ex2(s[n][0] - mu0), p1 = ex2(s[n][1] - mu0), p2 = ex2(s[n][2] - mu1), p3 = ex2(s[n][3] - mu1);
            rs0 += p0 + p1;
            rs1 += p2 + p3;
            const __nv_bfloat162 h01 = __floats2bfloat162_rn(p0, p1), h23 = __floats2bfloat162_rn(p2, p3);
            if constexpr (CW == 2) {
                const int col = (nb + n) * 8 + 2 * (lane & 3), ra = (lane >> 2) * PLD + col, rb = ((lane >> 2) + 8) * PLD + col;
                *reinterpret_cast<__nv_bfloat162*>(ph + ra) = h01;
                *reinterpret_cast<__nv_bfloat162*>(ph + rb) = h23;
                *reinterpret_cast<__nv_bfloat162*>(pl + ra) = __floats2bfloat162_rn(p0 - __low2float(h01), p1 - __high2float(h01));
                *reinterpret_cast<__nv_bfloat162*>(pl + rb) = __floats2bfloat162_rn(p2 - __low2float(h23), p3 - __high2float(h23));
            } else {
                const int kk = n >> 1, half = (n & 1) * 2;
                phi[kk][half] = *reinterpret_cast<const uint32_t*>(&h01);
                phi[kk][half + 1] = *reinterpret_cast<const uint32_t*>(&h23);
                plo[kk][half] = pack_bf16(p0 - __low2float(h01), p1 - __high2float(h01));
                plo[kk][half + 1] = pack_bf16(p2 - __low2float(h23), p3 - __high2float(h23));
            }
        }
        if constexpr (CW == 2) {
            pair_sync(rg);
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                ldsm_x4(phi[kk], ph + (lane & 15) * PLD + kk * 16 + (lane >> 4) * 8);
                ldsm_x4(plo[kk], pl + (lane & 15) * PLD + kk * 16 + (lane >> 4) * 8);
            }
        }
        l0 = l0 * al0 + rs0;                                     // per-thread part of the row sums; the quad meets at the end
        l1 = l1 * al1 + rs1;
#pragma unroll
        for (int i = 0; i < NO; ++i) {
            if (i < nct) { o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1; }
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
            for (int i = 0; i < NO; ++i) {
                if (i < nct) {
                    uint32_t bfr[2];
                    ldsm_x2_trans(bfr, kt + (kk * 16 + (lane & 15)) * srow + (cs * NO + i) * 8);
                    mma_bf16(o[i], phi[kk], bfr);
                    mma_bf16(o[i], plo[kk], bfr);
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if constexpr (CW == 2) {                                     // each warp of a pair has summed the weights of its own keys
        float* mine = Mx + (rg * 2 + cs) * 16;
        if ((lane & 3) == 0) { mine[lane >> 2] = l0; mine[8 + (lane >> 2)] = l1; }
        pair_sync(rg);
        const float* other = Mx + (rg * 2 + (cs ^ 1)) * 16;
        l0 += other[lane >> 2];
        l1 += other[8 + (lane >> 2)];
    }
    const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
#pragma unroll
    for (int i = 0; i < NO; ++i) {
        if (i < nct) {
            const int col = (cs * NO + i) * 8 + 2 * (lane & 3);
            if (r0 < rows)
                *reinterpret_cast<float2*>(out + ((size_t)(tok0 + r0) * H + h) * R + col) = make_float2(o[i][0] * inv0, o[i][1] * inv0);
            if (r0 + 8 < rows)
                *reinterpret_cast<float2*>(out + ((size_t)(tok0 + r0 + 8) * H + h) * R + col) = make_float2(o[i][2] * inv1, o[i][3] * inv1);
        }
    }
}

template <int NO, int CW, int QL>
int launch_mma_q(const float* qa, const void* pages, int row, const int* bt, int bt_stride, const int* tiles, int n_tiles,
               const int* positions, float* out, int H, int R, int dk, int ps, float scale, cudaStream_t stream) {
    const size_t smem = (size_t)((QL ? 2 : 1) * MQ + 2 * MK) * (dk + 8) * 2 + (CW == 2 ? PAIR_BYTES : 0);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        MLLM_CUDA(cudaFuncSetAttribute(latent_mma_kernel<NO, CW, QL>, cudaFuncAttributeMaxDynamicSharedMemorySize, MAX_SMEM));
        raised = true;
    }
    MLLM_CUDA(mllm_launch(latent_mma_kernel<NO, CW, QL>, dim3(H, n_tiles), dim3(128 * CW), smem, stream, true, qa,
                          (const __nv_bfloat16*)pages, row, bt, bt_stride, tiles, positions, out, H, R, dk, ps, scale));
    return 0;
}

template <int NO, int CW>
int launch_mma(const float* qa, const void* pages, int row, const int* bt, int bt_stride, const int* tiles, int n_tiles,
               const int* positions, float* out, int H, int R, int dk, int ps, float scale, cudaStream_t stream) {
    if ((size_t)(2 * MQ + 2 * MK) * (dk + 8) * 2 + (CW == 2 ? PAIR_BYTES : 0) <= MAX_SMEM)
        return launch_mma_q<NO, CW, 1>(qa, pages, row, bt, bt_stride, tiles, n_tiles, positions, out, H, R, dk, ps, scale, stream);
    return launch_mma_q<NO, CW, 0>(qa, pages, row, bt, bt_stride, tiles, n_tiles, positions, out, H, R, dk, ps, scale, stream);
}

// The per-head products of many tokens on tensor cores (bfloat16 weights): 64 tokens x 64 columns per CTA and head, K in
// steps of 64.  MODE 0: inputs in bfloat16 (cp.async), result 32-bit.  MODE 1: inputs 32-bit, taken as hi + lo bfloat16
// terms so that they keep about 16 bits; result bfloat16, optionally times sigmoid(gate).
template <int MODE>
__global__ void __launch_bounds__(128)
headwise_mma_kernel(const void* in_, long long ld_in, int in_head, const __nv_bfloat16* __restrict__ W, void* out_,
                    long long ld_out, int out_head, const __nv_bfloat16* gate, long long ld_gate, int Tn, int N, int K) {
    using bf = __nv_bfloat16;
    constexpr int LD = 72;
    __shared__ __align__(16) bf As[64 * LD];
    __shared__ __align__(16) bf Al[MODE ? 64 * LD : 8];
    __shared__ __align__(16) bf Ws[64 * LD];
    pdl_wait();
    const int h = blockIdx.z, t0 = blockIdx.x * 64, n0 = blockIdx.y * 64;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float acc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }
    for (int k0 = 0; k0 < K; k0 += 64) {
        __syncthreads();                                         // the tiles of the step before have been used
        for (int i = tid; i < 64 * 8; i += 128) {
            const int r = i >> 3, pc = i & 7, k = k0 + pc * 8;
            const bool ok = n0 + r < N && k < K;
            cp_async16(Ws + r * LD + pc * 8, ok ? W + ((size_t)h * N + n0 + r) * K + k : W, ok);
            if (MODE == 0) {
                const bf* in = reinterpret_cast<const bf*>(in_);
                const bool oka = t0 + r < Tn && k < K;
                cp_async16(As + r * LD + pc * 8, oka ? in + (size_t)(t0 + r) * ld_in + (size_t)h * in_head + k : in, oka);
            }
        }
        if (MODE == 1) {
            const float* in = reinterpret_cast<const float*>(in_);
            for (int i = tid; i < 64 * 32; i += 128) {
                const int r = i >> 5, k = k0 + 2 * (i & 31);
                float2 v = make_float2(0.f, 0.f);
                if (t0 + r < Tn && k < K) v = *reinterpret_cast<const float2*>(in + (size_t)(t0 + r) * ld_in + (size_t)h * in_head + k);
                const __nv_bfloat162 hi = __floats2bfloat162_rn(v.x, v.y);
                *reinterpret_cast<__nv_bfloat162*>(As + r * LD + 2 * (i & 31)) = hi;
                *reinterpret_cast<__nv_bfloat162*>(Al + r * LD + 2 * (i & 31)) = __floats2bfloat162_rn(v.x - __low2float(hi), v.y - __high2float(hi));
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 64; kk += 16) {
            uint32_t af[4], al[4];
            ldsm_x4(af, As + (warp * 16 + (lane & 15)) * LD + kk + (lane >> 4) * 8);
            if (MODE == 1) ldsm_x4(al, Al + (warp * 16 + (lane & 15)) * LD + kk + (lane >> 4) * 8);
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                uint32_t b[2];
                ldsm_x2(b, Ws + (n * 8 + (lane & 7)) * LD + kk + ((lane >> 3) & 1) * 8);
                mma_bf16(acc[n], af, b);
                if (MODE == 1) mma_bf16(acc[n], al, b);
            }
        }
    }
    const int r0 = warp * 16 + (lane >> 2);
#pragma unroll
    for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int t = t0 + r0 + (c >> 1) * 8, col = n0 + n * 8 + 2 * (lane & 3) + (c & 1);
            if (t < Tn && col < N) {
                float v = acc[n][c];
                if (MODE == 0) {
                    reinterpret_cast<float*>(out_)[(size_t)t * ld_out + (size_t)h * out_head + col] = v;
                } else {
                    if (gate) v *= 1.0f / (1.0f + expf(-to_f32(gate[(size_t)t * ld_gate + (size_t)h * N + col])));
                    reinterpret_cast<bf*>(out_)[(size_t)t * ld_out + (size_t)h * out_head + col] = __float2bfloat16_rn(v);
                }
            }
        }
    }
}

}  // namespace

// proj [T, ...] in `dtype` with row stride ld: queries at column q_off (H heads of dn + dr), the down-projection at
// dkv_off (R + dr columns; -1: this layer writes no cache row).  pages [slots][row] in `dtype`.  qa [T][H][R + dr] 32-bit:
// only its columns R.. are written here.
MLLM_EXPORT int mllm_latent_prepare(const void* proj, long long ld, int q_off, int dkv_off, int Tn, int H, int dn, int dr,
                                    int R, int rot_dims, const int* positions, const int* slot_mapping, const float* freq,
                                    float mscale, const float* normw, float eps, void* pages, int row, float* qa,
                                    int write, int dtype, cudaStream_t stream) {
    if (Tn <= 0) return 0;
    if (rot_dims < 0 || rot_dims > dr || rot_dims % 2) return mllm_fail(1, "latent_prepare: %d rotated dimensions of %d", rot_dims, dr);
    if (row < R + dr) return mllm_fail(1, "latent_prepare: cache rows of %d cannot hold %d + %d", row, R, dr);
    if (dtype == MLLM_F32)
        MLLM_CUDA(mllm_launch(latent_prepare_kernel<float>, dim3(Tn), dim3(128), 0, stream, true, (const float*)proj, ld, q_off,
                              dkv_off, H, dn, dr, R, rot_dims, positions, slot_mapping, freq, mscale, normw, eps,
                              (float*)pages, row, qa, write));
    else if (dtype == MLLM_BF16)
        MLLM_CUDA(mllm_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(Tn), dim3(128), 0, stream, true,
                              (const __nv_bfloat16*)proj, ld, q_off, dkv_off, H, dn, dr, R, rot_dims, positions, slot_mapping,
                              freq, mscale, normw, eps, (__nv_bfloat16*)pages, row, qa, write));
    else
        return mllm_fail(1, "latent_prepare: unknown dtype code %d", dtype);
    return 0;
}

// mode 0: in `dtype`, W `dtype`, out 32-bit (no gate).  mode 1: in 32-bit, W `dtype`, out `dtype`, optional gate in `dtype`.
MLLM_EXPORT int mllm_headwise_linear(const void* in, long long ld_in, int in_head, const void* W, void* out, long long ld_out,
                                     int out_head, const void* gate, long long ld_gate, int Tn, int H, int N, int K, int mode,
                                     int dtype, cudaStream_t stream) {
    if (Tn <= 0 || H <= 0 || N <= 0) return 0;
    if (K <= 0) return mllm_fail(1, "headwise_linear: K = %d", K);
    const dim3 grid((Tn + 31) / 32, (N + 63) / 64, H), block(256);
    if (grid.y > 65535 || grid.z > 65535) return mllm_fail(1, "headwise_linear: grid too large");
    if (mode == 0 && gate) return mllm_fail(1, "headwise_linear: a gate needs mode 1");
    if (Tn <= 16 && (size_t)K * 4 <= 48 * 1024 && H <= 65535) {                 // few tokens: every (token, head) streams its weights
        const dim3 rg(Tn, H, (N + 63) / 64);
        const size_t smem = (size_t)K * 4;
        if (dtype == MLLM_F32)
            MLLM_CUDA(mllm_launch(headwise_rows_kernel<float, float, float>, rg, block, smem, stream, true, (const float*)in, ld_in,
                                  in_head, (const float*)W, (float*)out, ld_out, out_head, (const float*)gate, ld_gate, N, K));
        else if (dtype == MLLM_BF16 && mode == 0)
            MLLM_CUDA(mllm_launch(headwise_rows_kernel<__nv_bfloat16, __nv_bfloat16, float>, rg, block, smem, stream, true,
                                  (const __nv_bfloat16*)in, ld_in, in_head, (const __nv_bfloat16*)W, (float*)out, ld_out, out_head,
                                  (const float*)nullptr, ld_gate, N, K));
        else if (dtype == MLLM_BF16)
            MLLM_CUDA(mllm_launch(headwise_rows_kernel<float, __nv_bfloat16, __nv_bfloat16>, rg, block, smem, stream, true,
                                  (const float*)in, ld_in, in_head, (const __nv_bfloat16*)W, (__nv_bfloat16*)out, ld_out, out_head,
                                  (const __nv_bfloat16*)gate, ld_gate, N, K));
        else
            return mllm_fail(1, "headwise_linear: unknown dtype code %d", dtype);
        return 0;
    }
    if (dtype == MLLM_BF16 && K % 8 == 0 && (uintptr_t)W % 16 == 0) {            // many tokens, bfloat16: tensor cores
        const dim3 mg((Tn + 63) / 64, (N + 63) / 64, H);
        if (mode == 0 && ld_in % 8 == 0 && in_head % 8 == 0 && (uintptr_t)in % 16 == 0) {
            MLLM_CUDA(mllm_launch(headwise_mma_kernel<0>, mg, dim3(128), 0, stream, true, in, ld_in, in_head, (const __nv_bfloat16*)W, out,
                                  ld_out, out_head, (const __nv_bfloat16*)nullptr, ld_gate, Tn, N, K));
            return 0;
        }
        if (mode == 1 && ld_in % 2 == 0 && in_head % 2 == 0 && (uintptr_t)in % 8 == 0) {
            MLLM_CUDA(mllm_launch(headwise_mma_kernel<1>, mg, dim3(128), 0, stream, true, in, ld_in, in_head, (const __nv_bfloat16*)W, out,
                                  ld_out, out_head, (const __nv_bfloat16*)gate, ld_gate, Tn, N, K));
            return 0;
        }
    }
    if (dtype == MLLM_F32) {
        MLLM_CUDA(mllm_launch(headwise_linear_kernel<float, float, float>, grid, block, 0, stream, true, (const float*)in, ld_in,
                              in_head, (const float*)W, (float*)out, ld_out, out_head, (const float*)gate, ld_gate, Tn, N, K));
    } else if (dtype == MLLM_BF16) {
        if (mode == 0)
            MLLM_CUDA(mllm_launch(headwise_linear_kernel<__nv_bfloat16, __nv_bfloat16, float>, grid, block, 0, stream, true,
                                  (const __nv_bfloat16*)in, ld_in, in_head, (const __nv_bfloat16*)W, (float*)out, ld_out,
                                  out_head, (const float*)nullptr, ld_gate, Tn, N, K));
        else
            MLLM_CUDA(mllm_launch(headwise_linear_kernel<float, __nv_bfloat16, __nv_bfloat16>, grid, block, 0, stream, true,
                                  (const float*)in, ld_in, in_head, (const __nv_bfloat16*)W, (__nv_bfloat16*)out, ld_out,
                                  out_head, (const __nv_bfloat16*)gate, ld_gate, Tn, N, K));
    } else {
        return mllm_fail(1, "headwise_linear: unknown dtype code %d", dtype);
    }
    return 0;
}

// qa [T][H][dk] 32-bit, pages [slots][row] in `dtype` (a token's row: R latent columns, then dk - R rotated key columns),
// out [T][H][R] 32-bit; part_o [T * H * nsplit * R], part_ml [T * H * nsplit * 2] scratch; nsplit >= ceil(longest context / span).
MLLM_EXPORT int mllm_latent_attention(const float* qa, const void* pages, int row, const int* block_table, int bt_stride,
                                      const int* token_seq, const int* positions, float* part_o, float* part_ml, int nsplit,
                                      float* out, int Tn, int H, int R, int dk, int ps, float scale, int span, int dtype,
                                      cudaStream_t stream) {
    if (Tn <= 0) return 0;
    if (R <= 0 || R > MAX_R || dk < R || dk > MAX_DK) return mllm_fail(1, "latent_attention: latent size %d (at most %d), key size %d (at most %d)", R, MAX_R, dk, MAX_DK);
    const int es = dtype == MLLM_F32 ? 4 : 2;
    if (row < dk || (row * es) % 16 != 0 || (uintptr_t)pages % 16 != 0) return mllm_fail(1, "latent_attention: cache rows of %d elements must hold %d and be multiples of 16 bytes", row, dk);
    if (Tn > 65535) return mllm_fail(1, "latent_attention: more than 65535 tokens in a step");
    if (span < 32 || span % 32) return mllm_fail(1, "latent_attention: a split of %d keys (a multiple of 32)", span);
    int rc;
    if (dtype == MLLM_F32)
        rc = pick_attention<float>(R, qa, pages, row, block_table, bt_stride, token_seq, positions, part_o, part_ml, nsplit, Tn,
                                   H, dk, ps, scale, span, stream);
    else if (dtype == MLLM_BF16)
        rc = pick_attention<__nv_bfloat16>(R, qa, pages, row, block_table, bt_stride, token_seq, positions, part_o, part_ml,
                                           nsplit, Tn, H, dk, ps, scale, span, stream);
    else
        return mllm_fail(1, "latent_attention: unknown dtype code %d", dtype);
    if (rc) return rc;
    MLLM_CUDA(mllm_launch(latent_merge_kernel, dim3((Tn * H + 7) / 8), dim3(256), 0, stream, true, part_o, part_ml, positions,
                          out, nsplit, Tn * H, H, R, span));
    return 0;
}

// 1 if the tensor-core kernel for prompt portions takes these sizes (a bfloat16 cache is the caller's to check).
MLLM_EXPORT int mllm_latent_mma_ok(int R, int dk, int row) {
    return R > 0 && R % 8 == 0 && R <= MAX_R && dk % 16 == 0 && dk >= R && row >= dk && row % 8 == 0 &&
           (size_t)(MQ + 2 * MK) * (dk + 8) * 2 + PAIR_BYTES <= MAX_SMEM;
}

// Prompt portions with a bfloat16 cache: tiles [n_tiles][3] = (request, first flat token, rows <= 64).
MLLM_EXPORT int mllm_latent_attention_mma(const float* qa, const void* pages, int row, const int* block_table, int bt_stride,
                                          const int* tiles, int n_tiles, const int* positions, float* out, int H, int R,
                                          int dk, int ps, float scale, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (!mllm_latent_mma_ok(R, dk, row) || (uintptr_t)pages % 16 != 0 || (uintptr_t)qa % 8 != 0)
        return mllm_fail(1, "latent_attention_mma: latent %d, key %d, row %d: not sizes this kernel takes", R, dk, row);
    if (n_tiles > 65535) return mllm_fail(1, "latent_attention_mma: too many tiles");
    if (R <= 32) return launch_mma<4, 1>(qa, pages, row, block_table, bt_stride, tiles, n_tiles, positions, out, H, R, dk, ps, scale, stream);
    if (R <= 64) return launch_mma<8, 1>(qa, pages, row, block_table, bt_stride, tiles, n_tiles, positions, out, H, R, dk, ps, scale, stream);
    if (R <= 128) return launch_mma<16, 1>(qa, pages, row, block_table, bt_stride, tiles, n_tiles, positions, out, H, R, dk, ps, scale, stream);
    if (R <= 256) return launch_mma<16, 2>(qa, pages, row, block_table, bt_stride, tiles, n_tiles, positions, out, H, R, dk, ps, scale, stream);
    if (R <= 384) return launch_mma<24, 2>(qa, pages, row, block_table, bt_stride, tiles, n_tiles, positions, out, H, R, dk, ps, scale, stream);
    return launch_mma<32, 2>(qa, pages, row, block_table, bt_stride, tiles, n_tiles, positions, out, H, R, dk, ps, scale, stream);
}
