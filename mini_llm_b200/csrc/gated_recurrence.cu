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

}  // namespace

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
