// Kernels of recurrent mixers with per-sequence state of fixed size: the short
// causal convolution in front of a state-space recurrence, the recurrence with a
// scalar decay per head (Mamba-2), and the gated RMS norm behind it.
//
// All of them serve a step of packed rows: sequence b owns rows
// cu_seqlens[b]..cu_seqlens[b+1], continues from the state kept for its cache
// slot, and leaves the state for its next step.  A prompt, a portion of one and
// a single token are the same case.  Decays, step sizes, the state, the sums of
// the recurrence and the norm are float whatever the activation type is.
#include "common.cuh"
#include <math.h>

namespace {

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
// log(1 + exp(x)) without overflow and without a cut-off
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// ------------------------------------------------ causal convolution + silu
// out[n, c] = silu(bias[c] + sum_j w[c, j] * in[n - (taps-1-j), c]): the last tap is
// the current token's.  Inputs before the first row of the step come from
// conv_state[slot, taps-1, C] (the sequence's last taps-1 inputs, oldest first;
// zero for a new sequence).  The sum runs in the same order however the
// sequence was cut into steps.
template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ in, int ld_in, const float* __restrict__ w,
                                        const float* __restrict__ bias, const float* __restrict__ conv_state,
                                        T* __restrict__ out, int ld_out, const int* __restrict__ token_seq,
                                        const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                                        int C, int taps) {
    chain_release();
    chain_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int n = blockIdx.x;
    const int b = token_seq[n];
    const int i = n - cu_seqlens[b];                 // rows of this sequence before n in the step
    const int keep = taps - 1;
    const float* st = conv_state + (size_t)slots[b] * keep * C;
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = keep - j;
        const float v = i - back >= 0 ? to_f32<T>(in[(size_t)(n - back) * ld_in + c])
                                      : st[(size_t)(keep + i - back) * C + c];
        acc = fmaf(w[(size_t)c * taps + j], v, acc);
    }
    out[(size_t)n * ld_out + c] = from_f32<T>(silu_f(acc));
}

// After the convolution: the state becomes the last taps-1 inputs of each
// sequence, the step's rows included.  One thread per (sequence, channel) walks
// oldest to newest, so a short step shifts the old entries without overtaking itself.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ in, int ld_in, float* __restrict__ conv_state,
                                         const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                                         int C, int taps) {
    chain_release();
    chain_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int b = blockIdx.y;
    const int first = cu_seqlens[b], len = cu_seqlens[b + 1] - first;
    const int keep = taps - 1;
    float* st = conv_state + (size_t)slots[b] * keep * C;
    for (int j = 0; j < keep; ++j) {
        const int src = len - keep + j;
        st[(size_t)j * C + c] = src >= 0 ? to_f32<T>(in[(size_t)(first + src) * ld_in + c])
                                         : st[(size_t)(j + len) * C + c];
    }
}

// ------------------------------------------- the recurrence, token by token
// Per head h (group g = h / (heads / groups)), with x_t [P], B_t, C_t [N], the
// step size dt_t = softplus(raw_t + dt_bias[h]) and the decay a_t = exp(-exp(a_log[h]) dt_t):
//     S_t = a_t S_{t-1} + dt_t B_t x_t^T          (S is N x P, float, kept per sequence)
//     y_t = S_t^T C_t + D[h] x_t
// One block per (head, sequence).  Thread (p, r) owns column p of S for the rows
// n = r, r + R, ...; the R partial sums of y_t[p] meet by shuffles.  Tokens are
// walked strictly in order, so the result does not depend on the cut of the
// sequence into steps nor on the batch.  x, B and C of kTile tokens at a time
// are staged in shared memory.
constexpr int kTile = 16;
constexpr int kRowsPerThread = 16;

template <typename T>
__global__ void ssm_scan_kernel(const T* __restrict__ xbc, int ld_xbc, const T* __restrict__ dt_raw, int ld_dt,
                                const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                const float* __restrict__ skip, float* __restrict__ state,
                                float* __restrict__ y, int ld_y, const int* __restrict__ cu_seqlens,
                                const int* __restrict__ slots, int heads, int groups, int N, int P, int R) {
    chain_release();
    chain_wait();
    extern __shared__ float smem[];
    float* sx = smem;                        // kTile * P
    float* sB = sx + kTile * P;              // kTile * N
    float* sC = sB + kTile * N;              // kTile * N
    float* sdt = sC + kTile * N;             // kTile
    float* sa = sdt + kTile;                 // kTile
    const int h = blockIdx.x, b = blockIdx.y;
    const int g = h / (heads / groups);
    const int inner = heads * P;
    const int tid = threadIdx.x;
    const int p = tid / R, r = tid - p * R;
    const bool owner = p < P;
    const int first = cu_seqlens[b], last = cu_seqlens[b + 1];
    float* S = state + ((size_t)slots[b] * heads + h) * N * P;
    float s[kRowsPerThread];
#pragma unroll
    for (int k = 0; k < kRowsPerThread; ++k) {
        const int n = r + R * k;
        s[k] = (owner && n < N) ? S[(size_t)n * P + p] : 0.f;
    }
    const float bias = dt_bias[h], rate = expf(a_log[h]), d_skip = skip[h];

    for (int t0 = first; t0 < last; t0 += kTile) {
        const int nt = min(kTile, last - t0);
        __syncthreads();
        for (int idx = tid; idx < nt * P; idx += blockDim.x) {
            const int tt = idx / P, pp = idx - tt * P;
            sx[idx] = to_f32<T>(xbc[(size_t)(t0 + tt) * ld_xbc + h * P + pp]);
        }
        for (int idx = tid; idx < nt * N; idx += blockDim.x) {
            const int tt = idx / N, nn = idx - tt * N;
            const T* row = xbc + (size_t)(t0 + tt) * ld_xbc + inner + g * N + nn;
            sB[idx] = to_f32<T>(row[0]);
            sC[idx] = to_f32<T>(row[groups * N]);
        }
        if (tid < nt) {
            const float dt = softplus_f(to_f32<T>(dt_raw[(size_t)(t0 + tid) * ld_dt + h]) + bias);
            sdt[tid] = dt;
            sa[tid] = expf(-rate * dt);
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float dt = sdt[tt], a = sa[tt];
            const float xv = owner ? sx[tt * P + p] : 0.f;
            const float dx = dt * xv;
            float acc = 0.f;
#pragma unroll
            for (int k = 0; k < kRowsPerThread; ++k) {
                const int n = r + R * k;
                if (n < N) {
                    s[k] = fmaf(a, s[k], sB[tt * N + n] * dx);
                    acc = fmaf(s[k], sC[tt * N + n], acc);
                }
            }
            for (int o = R >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (owner && r == 0) y[(size_t)(t0 + tt) * ld_y + h * P + p] = fmaf(d_skip, xv, acc);
        }
    }
    if (owner) {
#pragma unroll
        for (int k = 0; k < kRowsPerThread; ++k) {
            const int n = r + R * k;
            if (n < N) S[(size_t)n * P + p] = s[k];
        }
    }
}

// --------------------------------------------------- gate, then RMS norm
// v = y * silu(z); the row is cut into `parts` equal pieces and every piece is
// divided by its own root mean square (eps inside the root), then multiplied by
// the weight.  y float, z and out the activation type.  One block per (row, piece).
template <typename T>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ y, int ld_y, const T* __restrict__ z, int ld_z,
                                     const float* __restrict__ weight, float eps, T* __restrict__ out, int ld_out,
                                     int size) {
    chain_release();
    chain_wait();
    extern __shared__ float smem[];
    float* v = smem;                  // size floats
    float* scratch = smem + size;     // 33 floats
    const size_t n = blockIdx.x;
    const int c0 = blockIdx.y * size;
    float ss = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float val = y[n * ld_y + c0 + i] * silu_f(to_f32<T>(z[n * ld_z + c0 + i]));
        v[i] = val;
        ss += val * val;
    }
    const float total = block_sum(ss, scratch);
    const float s = 1.0f / sqrtf(total / (float)size + eps);
    for (int i = threadIdx.x; i < size; i += blockDim.x)
        out[n * ld_out + c0 + i] = from_f32<T>(v[i] * s * weight[c0 + i]);
}

}  // namespace

GTG_API int gtg_causal_conv_silu(int dtype, const void* in, int ld_in, const float* w, const float* bias,
                                 const float* conv_state, void* out, int ld_out, const int* token_seq,
                                 const int* cu_seqlens, const int* slots, int n_tokens, int C, int taps,
                                 cudaStream_t stream) {
    if (n_tokens <= 0 || C <= 0) return 0;
    if (taps < 1 || ld_in < C || ld_out < C || (taps > 1 && conv_state == nullptr)) return kErrBadArgument;
    if ((C + 127) / 128 > 65535) return kErrUnsupported;
    const dim3 grid(n_tokens, (C + 127) / 128);
    if (dtype == 0) return launch_chained(causal_conv_silu_kernel<float>, grid, dim3(128), 0, stream, (const float*)in, ld_in, w, bias, conv_state, (float*)out, ld_out, token_seq, cu_seqlens, slots, C, taps);
    if (dtype == 1) return launch_chained(causal_conv_silu_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)in, ld_in, w, bias, conv_state, (bf16*)out, ld_out, token_seq, cu_seqlens, slots, C, taps);
    return kErrBadArgument;
}

GTG_API int gtg_conv_state_update(int dtype, const void* in, int ld_in, float* conv_state, const int* cu_seqlens,
                                  const int* slots, int n_seqs, int C, int taps, cudaStream_t stream) {
    if (n_seqs <= 0 || C <= 0 || taps <= 1) return 0;
    if (n_seqs > 65535) return kErrUnsupported;
    const dim3 grid((C + 127) / 128, n_seqs);
    if (dtype == 0) return launch_chained(conv_state_update_kernel<float>, grid, dim3(128), 0, stream, (const float*)in, ld_in, conv_state, cu_seqlens, slots, C, taps);
    if (dtype == 1) return launch_chained(conv_state_update_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)in, ld_in, conv_state, cu_seqlens, slots, C, taps);
    return kErrBadArgument;
}

// How many threads share a column of the state: the least power of two that
// leaves a thread at most kRowsPerThread rows, widened while the block stays small.
static int scan_split(int N, int P) {
    int R = 1;
    while (R < 32 && (N + R - 1) / R > kRowsPerThread) R *= 2;
    while (R < 32 && R * 2 <= N && P * R * 2 <= 256) R *= 2;
    return R;
}

GTG_API int gtg_ssm_scan(int dtype, const void* xbc, int ld_xbc, const void* dt_raw, int ld_dt,
                         const float* dt_bias, const float* a_log, const float* skip, float* state,
                         float* y, int ld_y, const int* cu_seqlens, const int* slots, int n_seqs,
                         int heads, int groups, int N, int P, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (heads <= 0 || groups <= 0 || heads % groups || N <= 0 || P <= 0) return kErrBadArgument;
    if (n_seqs > 65535) return kErrUnsupported;
    const int R = scan_split(N, P);
    if ((N + R - 1) / R > kRowsPerThread) return kErrUnsupported;
    const int threads = (P * R + 31) / 32 * 32;
    if (threads > 1024) return kErrUnsupported;
    const size_t smem = (size_t)(kTile * (P + 2 * N) + 2 * kTile) * sizeof(float);
    if (smem > 200 * 1024) return kErrUnsupported;
    const dim3 grid(heads, n_seqs);
    cudaError_t e;
    if (dtype == 0) {
        if (smem > 48 * 1024 && (e = cudaFuncSetAttribute(ssm_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)e;
        return launch_chained(ssm_scan_kernel<float>, grid, dim3(threads), smem, stream, (const float*)xbc, ld_xbc, (const float*)dt_raw, ld_dt, dt_bias, a_log, skip, state, y, ld_y, cu_seqlens, slots, heads, groups, N, P, R);
    }
    if (dtype == 1) {
        if (smem > 48 * 1024 && (e = cudaFuncSetAttribute(ssm_scan_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)e;
        return launch_chained(ssm_scan_kernel<bf16>, grid, dim3(threads), smem, stream, (const bf16*)xbc, ld_xbc, (const bf16*)dt_raw, ld_dt, dt_bias, a_log, skip, state, y, ld_y, cu_seqlens, slots, heads, groups, N, P, R);
    }
    return kErrBadArgument;
}

GTG_API int gtg_gated_rmsnorm(int dtype, const float* y, int ld_y, const void* z, int ld_z, const float* weight,
                              float eps, void* out, int ld_out, int n_rows, int width, int parts,
                              cudaStream_t stream) {
    if (n_rows <= 0 || width <= 0) return 0;
    if (parts <= 0 || width % parts || parts > 65535) return kErrBadArgument;
    const int size = width / parts;
    int threads = 32;
    while (threads < 512 && threads * 2 < size) threads *= 2;
    const size_t smem = (size_t)(size + 33) * sizeof(float);
    if (smem > 200 * 1024) return kErrUnsupported;
    const dim3 grid(n_rows, parts);
    cudaError_t e;
    if (dtype == 0) {
        if (smem > 48 * 1024 && (e = cudaFuncSetAttribute(gated_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)e;
        return launch_chained(gated_rmsnorm_kernel<float>, grid, dim3(threads), smem, stream, y, ld_y, (const float*)z, ld_z, weight, eps, (float*)out, ld_out, size);
    }
    if (dtype == 1) {
        if (smem > 48 * 1024 && (e = cudaFuncSetAttribute(gated_rmsnorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)e;
        return launch_chained(gated_rmsnorm_kernel<bf16>, grid, dim3(threads), smem, stream, y, ld_y, (const bf16*)z, ld_z, weight, eps, (bf16*)out, ld_out, size);
    }
    return kErrBadArgument;
}
