// Mamba-2 (state-space duality) as three kernels around the projections:
//
//   conv_silu          the causal short convolution per channel over the step's tokens, with bias and silu; the taps - 1
//                      inputs before a portion come from the request's state (zero for a new request), so a prompt can
//                      be cut anywhere.  conv_state_update then stores the last taps - 1 inputs of every request.
//   ssd_scan           per request and head: dt = softplus(raw + bias), S <- exp(-exp(A_log) dt) S + dt B x^T,
//                      y = S^T C + D x, token by token.  A CTA owns 32 columns of a head's state S [N, P]; a warp owns 4
//                      columns, its lanes 8 row groups of consecutive rows, so a thread keeps N / 8 state elements
//                      in registers and the sum over rows ends in three shuffles.  Tokens are staged 16 at a time.
//                      Every state element is a recurrence of its own, so the state after n tokens is the same bits
//                      however the n tokens were cut into steps.
//   gated_group_norm   out = rms_norm_in_groups(y * silu(z)) * w.
// Everything here is 32-bit: the state, dt, the decay, the products; inputs come in the activation dtype.
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 16;
constexpr int CHUNK = 16;

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }
__device__ __forceinline__ void cp4(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}

// grid (channel blocks of 256, tokens).  u = proj[:, off : off + C]; state [slots][stride], the conv part at conv_off:
// [taps - 1][C], oldest first.
template <typename T>
__global__ void __launch_bounds__(256)
conv_silu_kernel(const T* proj, long long ld, int off, const float* __restrict__ w, const float* __restrict__ bias,
                 const float* state, long long state_stride, int conv_off, const int* token_seq, const int* cu_q,
                 const int* slots, float* out, int Tn, int C, int taps) {
    pdl_wait();
    const int t = blockIdx.y, ch = blockIdx.x * 256 + threadIdx.x;
    if (ch >= C) return;
    const int s = token_seq[t];
    const int qi = t - cu_q[s];
    float acc = bias[ch];
    if (qi >= taps - 1) {                   // every input lies in this step
        for (int j = 0; j < taps; ++j)
            acc = fmaf(w[(size_t)ch * taps + j], to_f32(proj[(size_t)(t - (taps - 1) + j) * ld + off + ch]), acc);
    } else {
        const float* st = state + (size_t)slots[s] * state_stride + conv_off;
        for (int j = 0; j < taps; ++j) {
            const int src = qi - (taps - 1) + j;
            const float u = src >= 0 ? to_f32(proj[(size_t)(t - (taps - 1) + j) * ld + off + ch])
                                     : st[(size_t)(taps - 1 + src) * C + ch];
            acc = fmaf(w[(size_t)ch * taps + j], u, acc);
        }
    }
    out[(size_t)t * C + ch] = silu_f(acc);
}

// Steps in which every request brings one token: grid (channel blocks, requests); a thread computes its channel's output
// from the state and the token, and shifts the token into the state (one launch instead of two).
template <typename T>
__global__ void __launch_bounds__(256)
conv_step_kernel(const T* proj, long long ld, int off, const float* __restrict__ w, const float* __restrict__ bias,
                 float* state, long long state_stride, int conv_off, const int* cu_q, const int* slots, float* out, int C,
                 int taps, int write_state) {
    pdl_wait();
    const int ch = blockIdx.x * 256 + threadIdx.x, s = blockIdx.y;
    if (ch >= C) return;
    const int t = cu_q[s];
    float* st = state + (size_t)slots[s] * state_stride + conv_off;
    const float u = to_f32(proj[(size_t)t * ld + off + ch]);
    float acc = bias[ch];
    float keep[MAX_TAPS];
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k) {
        if (k < taps - 1) {
            keep[k] = st[(size_t)k * C + ch];
            acc = fmaf(w[(size_t)ch * taps + k], keep[k], acc);
        }
    }
    acc = fmaf(w[(size_t)ch * taps + taps - 1], u, acc);
    out[(size_t)t * C + ch] = silu_f(acc);
    if (write_state) {
#pragma unroll
        for (int k = 0; k < MAX_TAPS; ++k) {
            if (k + 1 < taps - 1) st[(size_t)k * C + ch] = keep[k + 1];
            else if (k + 1 == taps - 1) st[(size_t)k * C + ch] = u;
        }
    }
}

// grid (channel blocks, requests): the state's conv part becomes the last taps - 1 inputs of the request.
template <typename T>
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const T* proj, long long ld, int off, float* state, long long state_stride, int conv_off,
                         const int* cu_q, const int* slots, int C, int taps) {
    pdl_wait();
    const int ch = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
    if (ch >= C) return;
    const int t0 = cu_q[s], n = cu_q[s + 1] - t0;
    float* st = state + (size_t)slots[s] * state_stride + conv_off;
    float keep[MAX_TAPS];
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k) {
        if (k < taps - 1) {
            const int idx = n - (taps - 1) + k;
            keep[k] = idx >= 0 ? to_f32(proj[(size_t)(t0 + idx) * ld + off + ch]) : st[(size_t)(k + n) * C + ch];
        }
    }
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k)
        if (k < taps - 1) st[(size_t)k * C + ch] = keep[k];
}

// grid (column blocks of 32, heads, requests), 256 threads.  xbc [T][C] 32-bit (x at 0, B at b_off, C at c_off);
// dt_raw = proj[:, dt_off + head] in the activation dtype; state [slots][stride] with S of head h at h * N * P, [N][P].
// Thread (column, rg) owns the ROWS consecutive state rows rg * ROWS ..: it reads its part of B_t and C_t with 16-byte
// loads (a token's B and C are staged with 4 floats of padding after every ROWS rows, so the eight row groups fall on
// different banks; rows beyond N are staged as zeros and stay zero in the state).
template <typename T, int ROWS>
__global__ void __launch_bounds__(256)
ssd_scan_kernel(const float* xbc, int Cw, int b_off, int c_off, const T* proj, long long ld, int dt_off,
                const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ Dh,
                float* state, long long state_stride, const int* cu_q, const int* slots, float* y, int Hm, int N, int P,
                int G, int write_state) {
    constexpr int PAD = ROWS == 4 ? 0 : 4;
    constexpr int NP = 8 * (ROWS + PAD);    // floats of a token's B (or C) in shared memory
    extern __shared__ __align__(16) float sm[];
    // two buffers of: B [CHUNK][NP], C [CHUNK][NP], x [CHUNK][32], dt [CHUNK], decay [CHUNK]
    pdl_wait();
    const int h = blockIdx.y, s = blockIdx.z, j0 = blockIdx.x * 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = j0 + warp * 4 + (lane >> 3), rg = lane & 7;
    const int g = h / (Hm / G);
    const int t0 = cu_q[s], n = cu_q[s + 1] - t0;
    float* S = state + (size_t)slots[s] * state_stride + (size_t)h * N * P;
    const bool live = col < P;
    float st[ROWS];
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
        const int r = rg * ROWS + i;
        st[i] = (live && r < N) ? S[(size_t)r * P + col] : 0.f;
    }
    const float a = -expf(A_log[h]), dskip = Dh[h], dtb = dt_bias[h];
    constexpr int BUF = 2 * CHUNK * NP + CHUNK * 32 + 2 * CHUNK;     // floats of one chunk's buffer
    // a chunk's B, C and x come in by 4-byte cp.async while the chunk before it is walked; its step sizes are read into
    // a register at the same time and turned into dt and the decay after the walk
    float raw_dt = 0.f;
    auto stage = [&](int c0, int buf) {
        const int nc = min(CHUNK, n - c0);
        float* B2 = sm + buf * BUF;
        float* C2 = B2 + CHUNK * NP;
        float* x2 = C2 + CHUNK * NP;
        for (int i = threadIdx.x; i < nc * 8 * ROWS; i += 256) {
            const int tt = i / (8 * ROWS), r = i - tt * 8 * ROWS;
            const float* rowp = xbc + (size_t)(t0 + c0 + tt) * Cw;
            const int at = tt * NP + r + (r / ROWS) * PAD;
            if (r < N) {
                cp4(B2 + at, rowp + b_off + g * N + r);
                cp4(C2 + at, rowp + c_off + g * N + r);
            } else {
                B2[at] = 0.f;
                C2[at] = 0.f;
            }
        }
        for (int i = threadIdx.x; i < nc * 32; i += 256) {
            const int tt = i >> 5, c = i & 31;
            if (j0 + c < P) cp4(x2 + i, xbc + (size_t)(t0 + c0 + tt) * Cw + (size_t)h * P + j0 + c);
            else x2[i] = 0.f;
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (threadIdx.x < nc) raw_dt = to_f32(proj[(size_t)(t0 + c0 + threadIdx.x) * ld + dt_off + h]);
    };
    auto steps = [&](int c0, int buf) {
        if (threadIdx.x < min(CHUNK, n - c0)) {
            float* d2 = sm + buf * BUF + 2 * CHUNK * NP + CHUNK * 32;
            const float dt = softplus_f(raw_dt + dtb);
            d2[threadIdx.x] = dt;
            d2[CHUNK + threadIdx.x] = expf(a * dt);
        }
    };
    if (n > 0) {
        stage(0, 0);
        steps(0, 0);
    }
    for (int c0 = 0, buf = 0; c0 < n; c0 += CHUNK, buf ^= 1) {
        const int nc = min(CHUNK, n - c0);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                    // this chunk is in; the other buffer has been walked
        const bool more = c0 + CHUNK < n;
        if (more) stage(c0 + CHUNK, buf ^ 1);
        const float* Bs = sm + buf * BUF;
        const float* Cs = Bs + CHUNK * NP;
        const float* xs = Cs + CHUNK * NP;
        const float* dts = xs + CHUNK * 32;
        const float* das = dts + CHUNK;
        for (int tt = 0; tt < nc; ++tt) {
            const float dt = dts[tt], da = das[tt], xv = xs[tt * 32 + warp * 4 + (lane >> 3)];
            const float dx = dt * xv;
            const float4* Bt = reinterpret_cast<const float4*>(Bs + tt * NP + rg * (ROWS + PAD));
            const float4* Ct = reinterpret_cast<const float4*>(Cs + tt * NP + rg * (ROWS + PAD));
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;        // four partial sums: the order is fixed, the chain short
#pragma unroll
            for (int i = 0; i < ROWS / 4; ++i) {
                const float4 b = Bt[i], c = Ct[i];
                st[4 * i] = fmaf(da, st[4 * i], b.x * dx);
                a0 = fmaf(st[4 * i], c.x, a0);
                st[4 * i + 1] = fmaf(da, st[4 * i + 1], b.y * dx);
                a1 = fmaf(st[4 * i + 1], c.y, a1);
                st[4 * i + 2] = fmaf(da, st[4 * i + 2], b.z * dx);
                a2 = fmaf(st[4 * i + 2], c.z, a2);
                st[4 * i + 3] = fmaf(da, st[4 * i + 3], b.w * dx);
                a3 = fmaf(st[4 * i + 3], c.w, a3);
            }
            float acc = (a0 + a1) + (a2 + a3);
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (rg == 0 && live) y[(size_t)(t0 + c0 + tt) * ((size_t)Hm * P) + (size_t)h * P + col] = fmaf(dskip, xv, acc);
        }
        if (more) steps(c0 + CHUNK, buf ^ 1);
    }
    if (write_state && live) {
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
            const int r = rg * ROWS + i;
            if (r < N) S[(size_t)r * P + col] = st[i];
        }
    }
}

// grid (groups, tokens): out[t][g] = v / sqrt(mean(v^2) + eps) * w with v = y * silu(z) over the group's columns.
template <typename T>
__global__ void __launch_bounds__(128)
gated_group_norm_kernel(const float* y, const T* z, long long ldz, const float* __restrict__ w, T* out, long long ldo,
                        int width, int gw, float eps) {
    __shared__ float scratch[33];
    pdl_wait();
    const int t = blockIdx.y, c0 = blockIdx.x * gw;
    const float* yr = y + (size_t)t * width + c0;
    const T* zr = z + (size_t)t * ldz + c0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < gw; i += blockDim.x) {
        const float v = yr[i] * silu_f(to_f32(zr[i]));
        ss = fmaf(v, v, ss);
    }
    const float r = sqrtf(block_sum(ss, scratch) / (float)gw + eps);
    for (int i = threadIdx.x; i < gw; i += blockDim.x) {
        const float v = yr[i] * silu_f(to_f32(zr[i]));
        out[(size_t)t * ldo + c0 + i] = from_f32<T>(v / r * w[c0 + i]);
    }
}

template <typename T>
int scan_launch(int rows, dim3 grid, size_t smem, cudaStream_t stream, const float* xbc, int Cw, int b_off, int c_off,
                const void* proj, long long ld, int dt_off, const float* dt_bias, const float* A_log, const float* Dh,
                float* state, long long state_stride, const int* cu_q, const int* slots, float* y, int Hm, int N, int P, int G,
                int write_state) {
#define MLLM_SCAN(R)                                                                                                     \
    do {                                                                                                                 \
        static bool raised = false;                                                                                      \
        if (smem > 48 * 1024 && !raised) {                                                                               \
            MLLM_CUDA(cudaFuncSetAttribute(ssd_scan_kernel<T, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024)); \
            raised = true;                                                                                               \
        }                                                                                                                \
        MLLM_CUDA(mllm_launch(ssd_scan_kernel<T, R>, grid, dim3(256), smem, stream, true, xbc, Cw, b_off, c_off,         \
                              (const T*)proj, ld, dt_off, dt_bias, A_log, Dh, state, state_stride, cu_q, slots, y, Hm, N, P, \
                              G, write_state));                                                                          \
    } while (0)
    if (rows <= 4) MLLM_SCAN(4);
    else if (rows <= 8) MLLM_SCAN(8);
    else if (rows <= 16) MLLM_SCAN(16);
    else MLLM_SCAN(32);
#undef MLLM_SCAN
    return 0;
}

}  // namespace

MLLM_EXPORT int mllm_ssd_max_state_rows() { return 256; }
MLLM_EXPORT int mllm_ssd_max_taps() { return MAX_TAPS; }

// The convolution of the step's tokens (out [T][C] 32-bit), then the update of the requests' conv states.
MLLM_EXPORT int mllm_ssd_conv(const void* proj, long long ld, int off, const float* w, const float* bias, float* state,
                              long long state_stride, int conv_off, const int* token_seq, const int* cu_q, const int* slots,
                              float* out, int Tn, int S, int C, int taps, int write_state, int dtype, cudaStream_t stream) {
    if (Tn <= 0 || C <= 0) return 0;
    if (taps < 1 || taps > MAX_TAPS) return mllm_fail(1, "ssd_conv: %d taps (1 to %d)", taps, MAX_TAPS);
    if (Tn > 65535 || S > 65535) return mllm_fail(1, "ssd_conv: more than 65535 tokens in a step");
    const dim3 grid((C + 255) / 256, Tn);
    const dim3 ugrid((C + 255) / 256, S);
    const bool single = Tn == S;            // one token per request: output and state update in one launch
    if (dtype == MLLM_F32) {
        if (single) {
            MLLM_CUDA(mllm_launch(conv_step_kernel<float>, ugrid, dim3(256), 0, stream, true, (const float*)proj, ld, off, w, bias,
                                  state, state_stride, conv_off, cu_q, slots, out, C, taps, write_state));
            return 0;
        }
        MLLM_CUDA(mllm_launch(conv_silu_kernel<float>, grid, dim3(256), 0, stream, true, (const float*)proj, ld, off, w, bias,
                              (const float*)state, state_stride, conv_off, token_seq, cu_q, slots, out, Tn, C, taps));
        if (write_state && taps > 1)
            MLLM_CUDA(mllm_launch(conv_state_update_kernel<float>, ugrid, dim3(256), 0, stream, true, (const float*)proj, ld, off,
                                  state, state_stride, conv_off, cu_q, slots, C, taps));
    } else if (dtype == MLLM_BF16) {
        if (single) {
            MLLM_CUDA(mllm_launch(conv_step_kernel<__nv_bfloat16>, ugrid, dim3(256), 0, stream, true, (const __nv_bfloat16*)proj, ld,
                                  off, w, bias, state, state_stride, conv_off, cu_q, slots, out, C, taps, write_state));
            return 0;
        }
        MLLM_CUDA(mllm_launch(conv_silu_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, true, (const __nv_bfloat16*)proj,
                              ld, off, w, bias, (const float*)state, state_stride, conv_off, token_seq, cu_q, slots, out, Tn, C,
                              taps));
        if (write_state && taps > 1)
            MLLM_CUDA(mllm_launch(conv_state_update_kernel<__nv_bfloat16>, ugrid, dim3(256), 0, stream, true,
                                  (const __nv_bfloat16*)proj, ld, off, state, state_stride, conv_off, cu_q, slots, C, taps));
    } else {
        return mllm_fail(1, "ssd_conv: unknown dtype code %d", dtype);
    }
    return 0;
}

MLLM_EXPORT int mllm_ssd_scan(const float* xbc, int Cw, int b_off, int c_off, const void* proj, long long ld, int dt_off,
                              const float* dt_bias, const float* A_log, const float* Dh, float* state, long long state_stride,
                              const int* cu_q, const int* slots, float* y, int S, int Hm, int N, int P, int G, int write_state,
                              int dtype, cudaStream_t stream) {
    if (S <= 0) return 0;
    if (N < 1 || N > 256) return mllm_fail(1, "ssd_scan: a state of %d rows (1 to 256)", N);
    if (G < 1 || Hm % G) return mllm_fail(1, "ssd_scan: %d heads in %d groups", Hm, G);
    if (S > 65535 || Hm > 65535) return mllm_fail(1, "ssd_scan: grid too large");
    const dim3 grid((P + 31) / 32, Hm, S);
    const int rows = (N + 7) / 8;
    const int rpt = rows <= 4 ? 4 : rows <= 8 ? 8 : rows <= 16 ? 16 : 32;            // the instantiation's rows per thread
    const size_t smem = 2 * ((size_t)2 * CHUNK * 8 * (rpt + (rpt == 4 ? 0 : 4)) + CHUNK * 32 + 2 * CHUNK) * sizeof(float);
    if (dtype == MLLM_F32)
        return scan_launch<float>(rows, grid, smem, stream, xbc, Cw, b_off, c_off, proj, ld, dt_off, dt_bias, A_log, Dh, state,
                                  state_stride, cu_q, slots, y, Hm, N, P, G, write_state);
    if (dtype == MLLM_BF16)
        return scan_launch<__nv_bfloat16>(rows, grid, smem, stream, xbc, Cw, b_off, c_off, proj, ld, dt_off, dt_bias, A_log, Dh,
                                          state, state_stride, cu_q, slots, y, Hm, N, P, G, write_state);
    return mllm_fail(1, "ssd_scan: unknown dtype code %d", dtype);
}

MLLM_EXPORT int mllm_gated_group_norm(const float* y, const void* z, long long ldz, const float* w, void* out, long long ldo,
                                      int Tn, int width, int groups, float eps, int dtype, cudaStream_t stream) {
    if (Tn <= 0) return 0;
    if (groups < 1 || width % groups) return mllm_fail(1, "gated_group_norm: %d columns in %d groups", width, groups);
    if (Tn > 65535) return mllm_fail(1, "gated_group_norm: more than 65535 tokens in a step");
    const dim3 grid(groups, Tn);
    if (dtype == MLLM_F32)
        MLLM_CUDA(mllm_launch(gated_group_norm_kernel<float>, grid, dim3(128), 0, stream, true, y, (const float*)z, ldz, w,
                              (float*)out, ldo, width, width / groups, eps));
    else if (dtype == MLLM_BF16)
        MLLM_CUDA(mllm_launch(gated_group_norm_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, true, y, (const __nv_bfloat16*)z,
                              ldz, w, (__nv_bfloat16*)out, ldo, width, width / groups, eps));
    else
        return mllm_fail(1, "gated_group_norm: unknown dtype code %d", dtype);
    return 0;
}
