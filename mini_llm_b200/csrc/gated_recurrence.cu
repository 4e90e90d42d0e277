// A gated linear recurrence with a matrix state per head, whose forget gate also sets what is written:
//   f_t = lower + (1 - lower) * sigmoid(z_t + bias)            per head and row channel i (ek of them)
//   S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T                  S: [ek, ev] per head
//   o_t = S_t^T q_t,  q_t = silu(a_t)                           a: the query projection as the product left it
//   y_t = out_scale * o_t / sqrt(mean(o_t^2) + eps) * w         RMS norm over the head's ev outputs, w shared by heads
// The state is 32-bit and lives in a per-request slot; gates, their complements, the state update, o and the norm
// are 32-bit whatever the dtype of a, z, v and y.
//
// One CTA takes one (request, head) and walks the request's tokens of this step in order.  Thread (g, j) keeps rows
// g*RK .. g*RK+RK-1 of column j of the state in registers for the whole walk (the state is read once and written
// once per step).  Tokens are taken CH at a time: q and f of the chunk are computed once into shared memory, v of
// the chunk is staged, then every thread runs CH * RK fused multiply-adds without a barrier; the partial outputs of
// the row groups meet in shared memory and the warps share the chunk's tokens for the norm.  The order of every sum
// depends on the sizes only, never on how the tokens were cut into steps.
//
// That kernel suits steps of single tokens, where reading and writing the state is all the work.  For prompt portions
// a second kernel (`wide`) spreads one (request, head) over many more threads, since every element of the state is a
// recurrence of its own: a CTA takes 32 columns of the state, thread (g, j) keeps two or four rows of column j, so a
// token costs a thread two or four dependent fused multiply-adds instead of 64; the 32 tokens of a chunk are fetched into
// registers in one burst before anything is stored (loads and stores in one loop would be serialised, since the
// compiler cannot tell the global inputs from shared memory), and the raw outputs o_t go to a 32-bit buffer that the
// RMS norm kernel (csrc/rmsnorm.cu, one row per token and head) finishes.  Both kernels run the same recurrence per
// state element in the same order, so the state they leave is the same bit for bit.
#include "common.cuh"

namespace {

constexpr int RK = 64;              // rows of the state a thread keeps

struct RecArgs {
    const int* cu_q;        // [S+1] first flat token of every request of the step
    const int* slots;       // [S] state slot of every request
    const float* f_bias;    // [Hr*ek]
    const float* lower;     // [Hr*ek]
    const float* norm_w;    // [ev]
    float* state;           // [slots][Hr][ek][ev]
    long long a_stride, z_stride, v_stride, y_stride;
    int Hr, ek, ev, evp, groups, chunk, write_state;
    float eps, out_scale;
};

template <typename T>
__global__ void __launch_bounds__(512)
gated_recurrence_kernel(const T* a, const T* z, const T* v, T* __restrict__ y, RecArgs r) {
    extern __shared__ float sm[];
    const int ek = r.ek, ev = r.ev, CH = r.chunk, G = r.groups;
    float* qs = sm;                         // [CH][ek]
    float* fs = qs + CH * ek;               // [CH][ek]
    float* vs = fs + CH * ek;               // [CH][ev]
    float* os = vs + CH * ev;               // [G][CH][ev]
    pdl_wait();
    pdl_launch();
    const int seq = blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, j = tid % r.evp, g = tid / r.evp;
    const int t0 = r.cu_q[seq], t1 = r.cu_q[seq + 1];
    const int slot = r.slots[seq];
    const bool col = j < ev && g < G;
    const int i0 = g * RK;
    float* sp = r.state + (((size_t)slot * r.Hr + h) * ek) * ev + j;
    float s[RK];
#pragma unroll
    for (int i = 0; i < RK; ++i) s[i] = (col && i0 + i < ek) ? sp[(size_t)(i0 + i) * ev] : 0.f;
    const int nthreads = blockDim.x, warp = tid >> 5, lane = tid & 31, nwarp = nthreads >> 5;

    for (int c0 = t0; c0 < t1; c0 += CH) {
        const int n = min(CH, t1 - c0);
        __syncthreads();                    // the chunk before is no longer read
        for (int idx = tid; idx < n * ek; idx += nthreads) {
            const int c = idx / ek, i = idx % ek;
            const float av = to_f32(a[(size_t)(c0 + c) * r.a_stride + (size_t)h * ek + i]);
            const float zv = to_f32(z[(size_t)(c0 + c) * r.z_stride + (size_t)h * ek + i]) + r.f_bias[h * ek + i];
            const float lo = r.lower[h * ek + i];
            qs[c * ek + i] = av / (1.0f + expf(-av));
            fs[c * ek + i] = lo + (1.0f - lo) * (1.0f / (1.0f + expf(-zv)));
        }
        for (int idx = tid; idx < n * ev; idx += nthreads) {
            const int c = idx / ev, d = idx % ev;
            vs[c * ev + d] = to_f32(v[(size_t)(c0 + c) * r.v_stride + (size_t)h * ev + d]);
        }
        __syncthreads();
        if (col) {
            for (int c = 0; c < n; ++c) {
                const float vv = vs[c * ev + j];
                const float* fq = fs + c * ek + i0;
                const float* qq = qs + c * ek + i0;
                float o = 0.f;
#pragma unroll
                for (int i = 0; i < RK; ++i) {
                    if (i0 + i < ek) {
                        const float f = fq[i];
                        s[i] = fmaf(f, s[i], (1.0f - f) * vv);
                        o = fmaf(s[i], qq[i], o);
                    }
                }
                os[(g * CH + c) * ev + j] = o;
            }
        }
        __syncthreads();
        // the norm: warp w takes tokens w, w + nwarp, ...; row groups meet in group order
        for (int c = warp; c < n; c += nwarp) {
            float q2 = 0.f;
            for (int d = lane; d < ev; d += 32) {
                float o = os[c * ev + d];
                for (int gg = 1; gg < G; ++gg) o += os[(gg * CH + c) * ev + d];
                os[c * ev + d] = o;
                q2 = fmaf(o, o, q2);
            }
            const float inv = r.out_scale / sqrtf(warp_sum(q2) / (float)ev + r.eps);
            T* yr = y + (size_t)(c0 + c) * r.y_stride + (size_t)h * ev;
            for (int d = lane; d < ev; d += 32) yr[d] = from_f32<T>(os[c * ev + d] * inv * r.norm_w[d]);
        }
    }
    if (r.write_state && col) {
#pragma unroll
        for (int i = 0; i < RK; ++i)
            if (i0 + i < ek) sp[(size_t)(i0 + i) * ev] = s[i];
    }
}

// ---------------------------------------------------------------------------------------------------------------
// rows of the state a thread of the wide kernel keeps: template parameter WR, 2 (states of up to 64 rows: twice the
// warps to hide the walk's latencies) or 4 (up to 128 rows)
constexpr int WC = 32;              // columns of the state a CTA of the wide kernel takes
constexpr int WCH = 32;             // tokens per chunk
constexpr int WLD = 4;              // elements of a and of z that a thread fetches per chunk (32 * 4G / 32G)
constexpr int WVMAX = 8;            // elements of v a thread fetches ahead at most (32 / G of them: G >= 4)

// grid (requests, heads, ceil(ev / 32)); block (32, G) with G = ceil(ek / 4) row groups.  o [T][Hr*ev] float.
template <int WR> struct RowVec;
template <> struct RowVec<2> { using type = float2; };
template <> struct RowVec<4> { using type = float4; };

template <typename T, int WR>
__global__ void __launch_bounds__(1024)
gated_recurrence_wide_kernel(const T* a, const T* z, const T* v, float* __restrict__ o, long long o_stride, RecArgs r) {
    extern __shared__ __align__(16) float sm[];
    const int ek = r.ek, ev = r.ev, G = blockDim.y;
    const int ekp = G * WR;                   // rows padded to a multiple of 4: the padding has f = 1, q = 0
    float* qs = sm;                           // [WCH][ekp]
    float* fs = qs + WCH * ekp;               // [WCH][ekp]
    float* vs = fs + WCH * ekp;               // [WCH][WC]
    float* os = vs + WCH * WC;                // [G][WCH][WC]
    pdl_wait();
    pdl_launch();
    const int seq = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * WC;
    const int lane = threadIdx.x, g = threadIdx.y, tid = g * 32 + lane, nthreads = G * 32;
    const int t0 = r.cu_q[seq], t1 = r.cu_q[seq + 1];
    const int slot = r.slots[seq];
    const int j = j0 + lane;
    const bool col = j < ev;
    float* sp = r.state + (((size_t)slot * r.Hr + h) * ek) * ev + j;
    float s[WR];
#pragma unroll
    for (int i = 0; i < WR; ++i) s[i] = (col && g * WR + i < ek) ? sp[(size_t)(g * WR + i) * ev] : 0.f;

    // Every thread owns WLD elements of a chunk's a and z (32 * ekp = 4 * threads of them) and VPT = 32 / G of its v:
    // they are fetched into registers a chunk ahead, while the chunk before is being walked.
    const int VPT = (WCH * WC + nthreads - 1) / nthreads;       // at most WVMAX when G >= 32 / WVMAX
    const bool ahead = VPT <= WVMAX;
    float av[WLD], zv[WLD], vv_next[WVMAX];
    // where this thread's elements of a chunk lie, relative to the chunk's first token: the same in every chunk
    int a_off[WLD], z_off[WLD], v_off[WVMAX];                  // at most 32 rows of the step ahead: they fit an int
    int a_tok[WLD], v_tok[WVMAX];
#pragma unroll
    for (int u = 0; u < WLD; ++u) {
        const int idx = tid + u * nthreads, c = idx / ekp, i = idx % ekp;
        a_tok[u] = i < ek ? c : WCH;                             // WCH: never fetched (padding row)
        a_off[u] = (int)(c * r.a_stride) + h * ek + i;
        z_off[u] = (int)(c * r.z_stride) + h * ek + i;
    }
#pragma unroll
    for (int u = 0; u < WVMAX; ++u) {
        const int idx = tid + u * nthreads, c = idx / WC, d = idx % WC;
        v_tok[u] = (u < VPT && j0 + d < ev) ? c : WCH;
        v_off[u] = (int)(c * r.v_stride) + h * ev + j0 + d;
    }
    auto fetch = [&](int c0) {
        const int n = min(WCH, t1 - c0);
        const T* ab = a + (size_t)c0 * r.a_stride;
        const T* zb = z + (size_t)c0 * r.z_stride;
        const T* vb = v + (size_t)c0 * r.v_stride;
#pragma unroll
        for (int u = 0; u < WLD; ++u) {
            av[u] = zv[u] = 0.f;
            if (a_tok[u] < n) {
                av[u] = to_f32(ab[a_off[u]]);
                zv[u] = to_f32(zb[z_off[u]]);
            }
        }
        if (ahead) {
#pragma unroll
            for (int u = 0; u < WVMAX; ++u) vv_next[u] = v_tok[u] < n ? to_f32(vb[v_off[u]]) : 0.f;
        }
    };
    // the gate's bias and lower bound of this thread's elements: the same rows in every chunk
    float lo_r[WLD], fb_r[WLD];
#pragma unroll
    for (int u = 0; u < WLD; ++u) {
        const int i = (tid + u * nthreads) % ekp;
        lo_r[u] = i < ek ? r.lower[h * ek + i] : 0.f;
        fb_r[u] = i < ek ? r.f_bias[h * ek + i] : 0.f;
    }
    if (t0 < t1) fetch(t0);
    for (int c0 = t0; c0 < t1; c0 += WCH) {
        const int n = min(WCH, t1 - c0);
        __syncthreads();                      // the chunk before is no longer read
#pragma unroll
        for (int u = 0; u < WLD; ++u) {
            const int idx = tid + u * nthreads, i = idx % ekp;
            if (idx >= n * ekp) continue;
            float qv = 0.f, fv = 1.f;
            if (i < ek) {
                const float lo = lo_r[u];
                qv = av[u] * __frcp_rn(1.0f + expf(-av[u]));
                fv = lo + (1.0f - lo) * __frcp_rn(1.0f + expf(-(zv[u] + fb_r[u])));
            }
            qs[idx] = qv;
            fs[idx] = fv;
        }
        if (ahead) {
#pragma unroll
            for (int u = 0; u < WVMAX; ++u) {
                const int idx = tid + u * nthreads;
                if (u < VPT && idx < n * WC) vs[idx] = vv_next[u];
            }
        } else {
            for (int base = tid; base < n * WC; base += nthreads * WLD) {
                float vv[WLD];
#pragma unroll
                for (int u = 0; u < WLD; ++u) {
                    const int idx = base + u * nthreads, c = idx / WC, d = idx % WC;
                    vv[u] = (idx < n * WC && j0 + d < ev) ? to_f32(v[(size_t)(c0 + c) * r.v_stride + (size_t)h * ev + j0 + d]) : 0.f;
                }
#pragma unroll
                for (int u = 0; u < WLD; ++u) {
                    const int idx = base + u * nthreads;
                    if (idx < n * WC) vs[idx] = vv[u];
                }
            }
        }
        if (c0 + WCH < t1) fetch(c0 + WCH);   // the next chunk's loads are in flight during this chunk's walk
        __syncthreads();
        // four tokens at a time: all twelve reads of shared memory first, then the arithmetic, then the four stores
        // (in one loop the compiler keeps every read behind the store before it: it cannot tell the arrays apart)
        using RV = typename RowVec<WR>::type;
        int c = 0;
        for (; c + 4 <= n; c += 4) {
            float vv[4];
            RV fr[4], qr[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                vv[u] = vs[(c + u) * WC + lane];
                fr[u] = *reinterpret_cast<const RV*>(fs + (c + u) * ekp + g * WR);
                qr[u] = *reinterpret_cast<const RV*>(qs + (c + u) * ekp + g * WR);
            }
            float ov[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float* f = reinterpret_cast<const float*>(&fr[u]);
                const float* q = reinterpret_cast<const float*>(&qr[u]);
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < WR; ++i) {
                    s[i] = fmaf(f[i], s[i], (1.0f - f[i]) * vv[u]);
                    acc = fmaf(s[i], q[i], acc);
                }
                ov[u] = acc;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) os[(g * WCH + c + u) * WC + lane] = ov[u];
        }
        for (; c < n; ++c) {
            const float vv = vs[c * WC + lane];
            const RV fr = *reinterpret_cast<const RV*>(fs + c * ekp + g * WR);
            const RV qr = *reinterpret_cast<const RV*>(qs + c * ekp + g * WR);
            const float* f = reinterpret_cast<const float*>(&fr);
            const float* q = reinterpret_cast<const float*>(&qr);
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < WR; ++i) {
                s[i] = fmaf(f[i], s[i], (1.0f - f[i]) * vv);
                acc = fmaf(s[i], q[i], acc);
            }
            os[(g * WCH + c) * WC + lane] = acc;
        }
        __syncthreads();
        for (int idx = tid; idx < n * WC; idx += nthreads) {          // row groups meet in group order
            const int c = idx / WC, d = idx % WC;
            float acc = os[c * WC + d];
#pragma unroll 8
            for (int gg = 1; gg < G; ++gg) acc += os[(gg * WCH + c) * WC + d];
            if (j0 + d < ev) o[(size_t)(c0 + c) * o_stride + (size_t)h * ev + j0 + d] = acc;
        }
    }
    if (r.write_state && col) {
#pragma unroll
        for (int i = 0; i < WR; ++i)
            if (g * WR + i < ek) sp[(size_t)(g * WR + i) * ev] = s[i];
    }
}

}  // namespace

// The recurrence alone for prompt portions: o [T][Hr*ev] (32-bit, un-normed).  ek up to 128.
MLLM_EXPORT int mllm_gated_recurrence_wide(const void* a, long long a_stride, const void* z, long long z_stride,
                                           const void* v, long long v_stride, const float* f_bias, const float* lower,
                                           float* state, const int* cu_q, const int* slots, float* o, long long o_stride,
                                           int S, int Hr, int ek, int ev, int write_state, int dtype, cudaStream_t stream) {
    if (S <= 0) return 0;
    if (ek <= 0 || ev <= 0 || Hr <= 0) return mllm_fail(1, "gated_recurrence: sizes %d x %d x %d", Hr, ek, ev);
    const int WR = ek <= 64 ? 2 : 4;      // measured at 32 rows: 171 us with 2 rows per thread, 190 with 1, 240 with 4
    const int G = (ek + WR - 1) / WR;
    if (G > 32) return mllm_fail(1, "gated_recurrence: the wide kernel takes states of up to %d rows, not %d", 32 * WR, ek);
    if (Hr > 65535 || (ev + WC - 1) / WC > 65535) return mllm_fail(1, "gated_recurrence: sizes exceed the grid");
    const size_t smem = sizeof(float) * ((size_t)2 * WCH * G * WR + WCH * WC + (size_t)G * WCH * WC);
    RecArgs r{cu_q, slots, f_bias, lower, nullptr, state, a_stride, z_stride, v_stride, 0,
              Hr, ek, ev, 0, G, WCH, write_state, 0.f, 1.f};
    const dim3 grid(S, Hr, (ev + WC - 1) / WC), block(32, G);
    using bf = __nv_bfloat16;
#define MLLM_WIDE(TT, RR)                                                                                              \
    do {                                                                                                               \
        MLLM_CUDA(cudaFuncSetAttribute(gated_recurrence_wide_kernel<TT, RR>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                       (int)smem));                                                                    \
        MLLM_CUDA(mllm_launch(gated_recurrence_wide_kernel<TT, RR>, grid, block, smem, stream, true, (const TT*)a,      \
                              (const TT*)z, (const TT*)v, o, o_stride, r));                                            \
    } while (0)
    if (dtype == MLLM_F32) {
        if (WR == 2) MLLM_WIDE(float, 2); else MLLM_WIDE(float, 4);
    } else if (dtype == MLLM_BF16) {
        if (WR == 2) MLLM_WIDE(bf, 2); else MLLM_WIDE(bf, 4);
    } else {
        return mllm_fail(1, "gated_recurrence: unknown dtype code %d", dtype);
    }
    return 0;
}

MLLM_EXPORT int mllm_gated_recurrence(const void* a, long long a_stride, const void* z, long long z_stride, const void* v,
                                      long long v_stride, const float* f_bias, const float* lower, const float* norm_w,
                                      float* state, const int* cu_q, const int* slots, void* y, long long y_stride, int S,
                                      int Hr, int ek, int ev, float eps, float out_scale, int write_state, int dtype,
                                      cudaStream_t stream) {
    if (S <= 0) return 0;
    if (ek <= 0 || ev <= 0 || Hr <= 0) return mllm_fail(1, "gated_recurrence: sizes %d x %d x %d", Hr, ek, ev);
    const int groups = (ek + RK - 1) / RK;
    const int evp = ((ev + 31) / 32) * 32;
    if ((long long)groups * evp > 512)
        return mllm_fail(1, "gated_recurrence: a state of %d x %d per head needs %d threads; a CTA of this kernel has 512", ek, ev, groups * evp);
    int chunk = 16;
    auto bytes = [&](int ch) { return sizeof(float) * (size_t)ch * (2 * (size_t)ek + (size_t)ev * (1 + groups)); };
    while (chunk > 1 && bytes(chunk) > 96 * 1024) chunk /= 2;
    const size_t smem = bytes(chunk);
    if (smem > 200 * 1024) return mllm_fail(1, "gated_recurrence: sizes %d x %d need %zu bytes of shared memory", ek, ev, smem);
    RecArgs r{cu_q, slots, f_bias, lower, norm_w, state, a_stride, z_stride, v_stride, y_stride,
              Hr, ek, ev, evp, groups, chunk, write_state, eps, out_scale};
    if (Hr > 65535) return mllm_fail(1, "gated_recurrence: %d heads exceed the grid", Hr);
    using bf = __nv_bfloat16;
    if (dtype == MLLM_F32) {
        if (smem > 48 * 1024)
            MLLM_CUDA(cudaFuncSetAttribute(gated_recurrence_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        MLLM_CUDA(mllm_launch(gated_recurrence_kernel<float>, dim3(S, Hr), dim3(groups * evp), smem, stream, true,
                              (const float*)a, (const float*)z, (const float*)v, (float*)y, r));
    } else if (dtype == MLLM_BF16) {
        if (smem > 48 * 1024)
            MLLM_CUDA(cudaFuncSetAttribute(gated_recurrence_kernel<bf>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        MLLM_CUDA(mllm_launch(gated_recurrence_kernel<bf>, dim3(S, Hr), dim3(groups * evp), smem, stream, true,
                              (const bf*)a, (const bf*)z, (const bf*)v, (bf*)y, r));
    } else {
        return mllm_fail(1, "gated_recurrence: unknown dtype code %d", dtype);
    }
    return 0;
}
