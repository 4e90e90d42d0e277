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
//   latent_attention one CTA per (split of 256 keys, token, block of 8 heads): key rows are staged once for all the
//                    heads of the block in chunks of 32 that start at multiples of 32 from position 0; a warp is a
//                    head, its lanes are the 32 keys for the scores and 32 latent columns at a time for the weighted
//                    sum; online softmax in 32-bit with expf.  Partial (o, m, l) per split, merged in split order by
//                    latent_merge.  Splits and chunks are fixed ranges of positions, so a token's sums run in the same
//                    order whether it came in a prompt portion, alone, or in a batch.
#include "common.cuh"

namespace {

constexpr int SPLIT = 256;      // keys per split
constexpr int HB = 8;           // heads (warps) per CTA
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

// grid (splits, tokens, head blocks); dynamic shared memory: HB * dk floats of queries, then 32 key rows of `kw` words.
template <typename T, int NACC>
__global__ void __launch_bounds__(HB * 32)
latent_attention_kernel(const float* qa, const T* pages, int row, const int* block_table, int bt_stride,
                        const int* token_seq, const int* positions, float* part_o, float* part_ml, int nsplit, int H,
                        int R, int dk, int ps, float scale, int kw) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* qs = reinterpret_cast<float*>(smem_raw);
    uint32_t* ks = reinterpret_cast<uint32_t*>(qs + HB * dk);
    pdl_wait();
    const int t = blockIdx.y, split = blockIdx.x;
    const int p = positions[t];
    const int k_lo = split * SPLIT;
    if (k_lo > p) return;
    const int k_hi = min(k_lo + SPLIT - 1, p);          // inclusive
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h0 = blockIdx.z * HB, h = h0 + warp;
    const int nh = min(HB, H - h0);
    for (int i = threadIdx.x; i < nh * dk; i += blockDim.x) qs[i] = qa[((size_t)t * H + h0) * dk + i];
    const int* bt = block_table + (size_t)token_seq[t] * bt_stride;
    const int vec_per_row = row * (int)sizeof(T) / 16;   // rows are padded to multiples of 16 bytes
    float m = -INFINITY, l = 0.f, acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    const float* q = qs + warp * dk;
    for (int base = k_lo; base <= k_hi; base += 32) {
        __syncthreads();            // the queries are in; the last chunk has been used
        const int nk = min(32, k_hi - base + 1);
        for (int i = threadIdx.x; i < nk * vec_per_row; i += blockDim.x) {
            const int j = i / vec_per_row, v = i % vec_per_row;
            const int pos = base + j;
            const T* src = pages + ((size_t)bt[pos / ps] * ps + pos % ps) * row;
            const uint4 x = *reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(src) + 16 * v);
            uint32_t* dst = ks + j * kw + v * 4;
            dst[0] = x.x; dst[1] = x.y; dst[2] = x.z; dst[3] = x.w;
        }
        __syncthreads();
        if (h >= H) continue;
        float s = -INFINITY;
        if (lane < nk) {
            const uint32_t* kr = ks + lane * kw;
            float d0 = 0.f, d1 = 0.f;
            if constexpr (sizeof(T) == 4) {
                int d = 0;
                for (; d + 1 < dk; d += 2) {
                    d0 = fmaf(q[d], __uint_as_float(kr[d]), d0);
                    d1 = fmaf(q[d + 1], __uint_as_float(kr[d + 1]), d1);
                }
                if (d < dk) d0 = fmaf(q[d], __uint_as_float(kr[d]), d0);
            } else {
                int d = 0;
                for (; d + 1 < dk; d += 2) {
                    const uint32_t w = kr[d >> 1];
                    d0 = fmaf(q[d], __uint_as_float(w << 16), d0);
                    d1 = fmaf(q[d + 1], __uint_as_float(w & 0xffff0000u), d1);
                }
                if (d < dk) d0 = fmaf(q[d], __uint_as_float(kr[d >> 1] << 16), d0);
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
        for (int j = 0; j < nk; ++j) {
            const float w = __shfl_sync(0xffffffffu, pj, j);
            const uint32_t* kr = ks + j * kw;
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                const int d = lane + 32 * i;
                if (d < R) {
                    float c;
                    if constexpr (sizeof(T) == 4) c = __uint_as_float(kr[d]);
                    else c = __uint_as_float((d & 1) ? (kr[d >> 1] & 0xffff0000u) : (kr[d >> 1] << 16));
                    acc[i] = fmaf(w, c, acc[i]);
                }
            }
        }
    }
    if (h >= H) return;
    const size_t o = ((size_t)t * H + h) * nsplit + split;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < R) part_o[o * R + d] = acc[i];
    }
    if (lane == 0) {
        part_ml[o * 2] = m;
        part_ml[o * 2 + 1] = l;
    }
}

// One warp per (token, head): out = sum_s o_s e^(m_s - M) / sum_s l_s e^(m_s - M) over the splits the token has.
__global__ void __launch_bounds__(256)
latent_merge_kernel(const float* part_o, const float* part_ml, const int* positions, float* out, int nsplit, int TH, int H,
                    int R) {
    pdl_wait();
    const int th = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (th >= TH) return;
    const int ns = positions[th / H] / SPLIT + 1;
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
                     int ps, float scale, cudaStream_t stream) {
    int kw = row * (int)sizeof(T) / 4;
    kw |= 1;                                        // an odd row stride in words: lanes read their rows without bank conflicts
    const size_t smem = (size_t)HB * dk * 4 + (size_t)32 * kw * 4;
    static bool raised = false;                     // once per instantiation
    if (smem > 48 * 1024 && !raised) {
        MLLM_CUDA(cudaFuncSetAttribute(latent_attention_kernel<T, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        raised = true;
    }
    if (smem > 200 * 1024) return mllm_fail(1, "latent_attention: rows of %d need %zu bytes of shared memory", dk, smem);
    MLLM_CUDA(mllm_launch(latent_attention_kernel<T, NACC>, dim3(nsplit, Tn, (H + HB - 1) / HB), dim3(HB * 32), smem, stream,
                          true, qa, (const T*)pages, row, bt, bt_stride, token_seq, positions, part_o, part_ml, nsplit, H,
                          R, dk, ps, scale, kw));
    return 0;
}

template <typename T>
int pick_attention(int R, const float* qa, const void* pages, int row, const int* bt, int bt_stride, const int* token_seq,
                   const int* positions, float* part_o, float* part_ml, int nsplit, int Tn, int H, int dk, int ps,
                   float scale, cudaStream_t stream) {
    if (R <= 128)
        return launch_attention<T, 4>(qa, pages, row, bt, bt_stride, token_seq, positions, part_o, part_ml, nsplit, Tn, H, R,
                                      dk, ps, scale, stream);
    if (R <= 256)
        return launch_attention<T, 8>(qa, pages, row, bt, bt_stride, token_seq, positions, part_o, part_ml, nsplit, Tn, H, R,
                                      dk, ps, scale, stream);
    return launch_attention<T, 16>(qa, pages, row, bt, bt_stride, token_seq, positions, part_o, part_ml, nsplit, Tn, H, R, dk,
                                   ps, scale, stream);
}

}  // namespace

MLLM_EXPORT int mllm_latent_split_keys() { return SPLIT; }

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
// out [T][H][R] 32-bit; part_o [T * H * nsplit * R], part_ml [T * H * nsplit * 2] scratch; nsplit >= ceil(longest context / 256).
MLLM_EXPORT int mllm_latent_attention(const float* qa, const void* pages, int row, const int* block_table, int bt_stride,
                                      const int* token_seq, const int* positions, float* part_o, float* part_ml, int nsplit,
                                      float* out, int Tn, int H, int R, int dk, int ps, float scale, int dtype,
                                      cudaStream_t stream) {
    if (Tn <= 0) return 0;
    if (R <= 0 || R > MAX_R || dk < R || dk > MAX_DK) return mllm_fail(1, "latent_attention: latent size %d (at most %d), key size %d (at most %d)", R, MAX_R, dk, MAX_DK);
    const int es = dtype == MLLM_F32 ? 4 : 2;
    if (row < dk || (row * es) % 16 != 0 || (uintptr_t)pages % 16 != 0) return mllm_fail(1, "latent_attention: cache rows of %d elements must hold %d and be multiples of 16 bytes", row, dk);
    if (Tn > 65535) return mllm_fail(1, "latent_attention: more than 65535 tokens in a step");
    int rc;
    if (dtype == MLLM_F32)
        rc = pick_attention<float>(R, qa, pages, row, block_table, bt_stride, token_seq, positions, part_o, part_ml, nsplit, Tn,
                                   H, dk, ps, scale, stream);
    else if (dtype == MLLM_BF16)
        rc = pick_attention<__nv_bfloat16>(R, qa, pages, row, block_table, bt_stride, token_seq, positions, part_o, part_ml,
                                           nsplit, Tn, H, dk, ps, scale, stream);
    else
        return mllm_fail(1, "latent_attention: unknown dtype code %d", dtype);
    if (rc) return rc;
    MLLM_CUDA(mllm_launch(latent_merge_kernel, dim3((Tn * H + 7) / 8), dim3(256), 0, stream, true, part_o, part_ml, positions,
                          out, nsplit, Tn * H, H, R));
    return 0;
}
