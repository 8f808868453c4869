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

// Where channel c >= n_plain of row n lands among the pairs: run U first, then V.
__device__ __forceinline__ size_t pair_index(size_t n, int c, int n_plain, int C) {
    const int half = (C - n_plain) >> 1, q = c - n_plain;
    return n * 2 * half + (q < half ? 2 * q : 2 * (q - half) + 1);
}
// log(1 + exp(x)) without overflow and without a cut-off
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// ------------------------------------------------ causal convolution + silu
// out[n, c] = silu(bias[c] + sum_j w[j, c] * in[n - (taps-1-j), c]): the last tap is
// the current token's; w is held tap by tap, [taps, C], so that neighbouring
// channels read neighbouring weights.  Inputs before the first row of the step come from
// conv_state[slot, taps-1, C] (the sequence's last taps-1 inputs, oldest first;
// zero for a new sequence).  The sum runs in the same order however the
// sequence was cut into steps.  The first n_plain channels go to `out`; the rest,
// two equal runs U and V (the B and C of a recurrence), go to `pairs` as float
// (U_q, V_q) side by side, [row][q][2], the form in which the recurrence reads
// them; pairs == nullptr: every channel goes to `out`.
template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ in, int ld_in, const float* __restrict__ w,
                                        const float* __restrict__ bias, const float* __restrict__ conv_state,
                                        T* __restrict__ out, int ld_out, const int* __restrict__ token_seq,
                                        const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                                        int C, int taps, int n_plain, float* __restrict__ pairs) {
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
        acc = fmaf(w[(size_t)j * C + c], v, acc);
    }
    if (c < n_plain) out[(size_t)n * ld_out + c] = from_f32<T>(silu_f(acc));
    else pairs[pair_index(n, c, n_plain, C)] = silu_f(acc);
}

// The same for bfloat16 rows of 16-byte aligned runs: a thread takes 8 neighbouring
// channels of one token with 16-byte accesses (same sum, same order).
__global__ void causal_conv_silu_bf16_vec_kernel(const bf16* __restrict__ in, int ld_in, const float* __restrict__ w,
                                                 const float* __restrict__ bias, const float* __restrict__ conv_state,
                                                 bf16* __restrict__ out, int ld_out, const int* __restrict__ token_seq,
                                                 const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                                                 int C, int taps, int n_plain, float* __restrict__ pairs) {
    chain_release();
    chain_wait();
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (c >= C) return;
    const int n = blockIdx.x;
    const int b = token_seq[n];
    const int i = n - cu_seqlens[b];
    const int keep = taps - 1;
    const float* st = conv_state + (size_t)slots[b] * keep * C;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = bias ? bias[c + e] : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = keep - j;
        float v[8];
        if (i - back >= 0) {
            const uint4 raw = *reinterpret_cast<const uint4*>(in + (size_t)(n - back) * ld_in + c);
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h2[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
        } else {
            const float4* sp = reinterpret_cast<const float4*>(st + (size_t)(keep + i - back) * C + c);
            const float4 a = sp[0], d = sp[1];
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = d.x; v[5] = d.y; v[6] = d.z; v[7] = d.w;
        }
        const float4* wp = reinterpret_cast<const float4*>(w + (size_t)j * C + c);
        const float4 w0 = wp[0], w1 = wp[1];
        const float wj[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(wj[e], v[e], acc[e]);
    }
    if (c >= n_plain) {                      // n_plain and the runs are multiples of 8: a thread's channels stay together
#pragma unroll
        for (int e = 0; e < 8; ++e) pairs[pair_index(n, c + e, n_plain, C)] = silu_f(acc[e]);
        return;
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(silu_f(acc[2 * e]), silu_f(acc[2 * e + 1]));
    *reinterpret_cast<uint4*>(out + (size_t)n * ld_out + c) = o;
}

// The same for a prompt in bfloat16: a thread takes 8 neighbouring channels through a run
// of kConvRun tokens, with its taps and the last TAPS-1 inputs in registers, so that
// every input is loaded once (16 bytes, all of a run's loads in flight together) and the
// taps once per run.  Where a new sequence
// begins inside the run the window is read afresh from that sequence's state.  The sum
// has the order of the kernels above: bias, then the taps oldest first.
constexpr int kConvRun = 8;
template <int TAPS>
__global__ void causal_conv_silu_bf16_run_kernel(const bf16* __restrict__ in, int ld_in, const float* __restrict__ w,
                                                 const float* __restrict__ bias, const float* __restrict__ conv_state,
                                                 bf16* __restrict__ out, int ld_out, const int* __restrict__ token_seq,
                                                 const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                                                 int n_tokens, int C, int n_plain, float* __restrict__ pairs) {
    chain_release();
    chain_wait();
    constexpr int keep = TAPS - 1;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (c >= C) return;
    const int n0 = blockIdx.x * kConvRun;
    float wt[TAPS][8], bs[8], win[keep > 0 ? keep : 1][8];
#pragma unroll
    for (int j = 0; j < TAPS; ++j) {
        const float4* wp = reinterpret_cast<const float4*>(w + (size_t)j * C + c);
        const float4 a = wp[0], d = wp[1];
        wt[j][0] = a.x; wt[j][1] = a.y; wt[j][2] = a.z; wt[j][3] = a.w; wt[j][4] = d.x; wt[j][5] = d.y; wt[j][6] = d.z; wt[j][7] = d.w;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) bs[e] = bias ? bias[c + e] : 0.f;
    auto widen = [](const uint4& raw, float* v) {
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h2[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
    };
    int seq = -1;
    const int n_end = min(n0 + kConvRun, n_tokens);
    // all of the run's inputs are asked for before the first is used
    uint4 raw[kConvRun];
    int seq_of[kConvRun];
#pragma unroll
    for (int t = 0; t < kConvRun; ++t) {
        const int n = min(n0 + t, n_tokens - 1);
        raw[t] = *reinterpret_cast<const uint4*>(in + (size_t)n * ld_in + c);
        seq_of[t] = token_seq[n];
    }
#pragma unroll
    for (int t = 0; t < kConvRun; ++t) {
        const int n = n0 + t;
        if (n >= n_end) break;
        const int b = seq_of[t];
        if (b != seq) {                                   // the run's first token, or a new sequence: fill the window
            seq = b;
            const int i = n - cu_seqlens[b];
            const float* st = conv_state + (size_t)slots[b] * keep * C;
#pragma unroll
            for (int j = 0; j < keep; ++j) {
                const int back = keep - j;
                if (i - back >= 0) {
                    widen(*reinterpret_cast<const uint4*>(in + (size_t)(n - back) * ld_in + c), win[j]);
                } else {
                    const float4* sp = reinterpret_cast<const float4*>(st + (size_t)(keep + i - back) * C + c);
                    const float4 a = sp[0], d = sp[1];
                    win[j][0] = a.x; win[j][1] = a.y; win[j][2] = a.z; win[j][3] = a.w;
                    win[j][4] = d.x; win[j][5] = d.y; win[j][6] = d.z; win[j][7] = d.w;
                }
            }
        }
        float cur[8], acc[8];
        widen(raw[t], cur);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float a = bs[e];
#pragma unroll
            for (int j = 0; j < keep; ++j) a = fmaf(wt[j][e], win[j][e], a);
            acc[e] = silu_f(fmaf(wt[keep][e], cur[e], a));
        }
#pragma unroll
        for (int j = 0; j + 1 < keep; ++j)
#pragma unroll
            for (int e = 0; e < 8; ++e) win[j][e] = win[j + 1][e];
        if (keep > 0) {
#pragma unroll
            for (int e = 0; e < 8; ++e) win[keep - 1][e] = cur[e];
        }
        if (c >= n_plain) {
#pragma unroll
            for (int e = 0; e < 8; ++e) pairs[pair_index(n, c + e, n_plain, C)] = acc[e];
        } else {
            uint4 o;
            __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
            *reinterpret_cast<uint4*>(out + (size_t)n * ld_out + c) = o;
        }
    }
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

// A step in which every sequence brings one token: convolution and state update
// in one kernel, one thread per (sequence, channel); the same sum in the same order.
template <typename T>
__global__ void causal_conv_step_kernel(const T* __restrict__ in, int ld_in, const float* __restrict__ w,
                                        const float* __restrict__ bias, float* __restrict__ conv_state,
                                        T* __restrict__ out, int ld_out, const int* __restrict__ slots,
                                        int C, int taps, int n_plain, float* __restrict__ pairs) {
    chain_release();
    chain_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int b = blockIdx.x;
    const int keep = taps - 1;
    float* st = conv_state + (size_t)slots[b] * keep * C;
    const float cur = to_f32<T>(in[(size_t)b * ld_in + c]);
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < keep; ++j) {
        const float v = st[(size_t)j * C + c];
        acc = fmaf(w[(size_t)j * C + c], v, acc);
        if (j > 0) st[(size_t)(j - 1) * C + c] = v;
    }
    acc = fmaf(w[(size_t)keep * C + c], cur, acc);
    if (keep > 0) st[(size_t)(keep - 1) * C + c] = cur;
    if (c < n_plain) out[(size_t)b * ld_out + c] = from_f32<T>(silu_f(acc));
    else pairs[pair_index(b, c, n_plain, C)] = silu_f(acc);
}

// ------------------------------------------- the recurrence, token by token
// Per head h (group g = h / (heads / groups)), with x_t [P], B_t, C_t [N], the
// step size dt_t = softplus(raw_t + dt_bias[h]) and the decay a_t = exp(-exp(a_log[h]) dt_t):
//     S_t = a_t S_{t-1} + dt_t B_t x_t^T          (S is N x P, float, kept per sequence)
//     y_t = S_t^T C_t + D[h] x_t
// The columns of S never meet, so one block serves (head, sequence, a slice of PS
// columns): the slices give a single long prompt enough blocks to fill the
// device.  Thread (p, r) owns column p for the rows n = r, r + R, ...; the R
// partial sums of y_t[p] meet by shuffles, four tokens' worth at a time so that
// their latencies overlap.  Tokens are walked strictly in order: the result does
// not depend on the cut of the sequence into steps, on the batch or on the slices.
// x, B and C of a tile of tokens at a time are staged in shared memory: kMaxTile for the
// usual state sizes (up to 256 rows), kPlainTile for the others (up to 512 rows).
constexpr int kMaxTile = 32;
constexpr int kPlainTile = 16;
constexpr int kRowsPerThread = 16;

__device__ __forceinline__ void copy_async_16(void* smem_dst, const void* gmem_src) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void copy_async_wait_all_but_one() { asm volatile("cp.async.wait_group 1;\n" ::: "memory"); }

// x: [row][heads * P] of T; bc: [row][groups * N] float pairs (B_n, C_n), as the
// convolution leaves them.  kAsync: the runs a block needs are 16-byte aligned and
// arrive one tile ahead by asynchronous copies, the pairs straight into the place
// the arithmetic reads them from; otherwise (odd sizes) they are read plainly when
// their tile begins.
// KR: rows of S a thread owns (R * KR >= N; the rows beyond N, if any, are skipped).
// RT: R known when compiling, with N = RT * KR (every offset into the staged pairs
// is then a constant), or 0: R and N as passed.
// CP: neighbouring columns of S a thread owns (the pairs it reads serve all of them).
template <typename T, bool kAsync, int KR, int RT, int CP>
__global__ void ssm_scan_kernel(const T* __restrict__ x, int ld_x, const float2* __restrict__ bc, int ld_bc,
                                const T* __restrict__ dt_raw, int ld_dt,
                                const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                const float* __restrict__ skip, float* __restrict__ state,
                                float* __restrict__ y, int ld_y, const int* __restrict__ cu_seqlens,
                                const int* __restrict__ slots, int heads, int groups, int N_, int P, int R_, int PS) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) float smem[];
    constexpr int kVec = 16 / (int)sizeof(T);
    const int R = RT ? RT : R_, N = RT ? RT * KR : N_;
    constexpr int kTile = RT ? kMaxTile : kPlainTile;        // tokens staged at a time
    float2* sBC = reinterpret_cast<float2*>(smem);          // two tiles of kTile * N pairs
    float* sx = smem + 4 * kTile * N;                       // kTile * PS
    float2* sda = reinterpret_cast<float2*>(sx + kTile * PS + ((kTile * PS) & 1));   // kTile pairs (dt, a)
    T* rawx = reinterpret_cast<T*>(sda + kTile);            // two tiles of kTile * PS (kAsync only)
    const int h = blockIdx.x, b = blockIdx.y, p0 = blockIdx.z * PS;
    const int cols = min(PS, P - p0);
    const int g = h / (heads / groups);
    const int tid = threadIdx.x;
    const int pg = tid / R, r = tid - pg * R;
    const int pl = pg * CP;                                  // the thread's first column within the slice
    const bool owner = pl < cols;                            // (with CP > 1 a slice's columns are a multiple of CP)
    const int p = p0 + pl;
    const int first = cu_seqlens[b], last = cu_seqlens[b + 1];
    float* S = state + ((size_t)slots[b] * heads + h) * N * P;
    float s[CP][KR];
#pragma unroll
    for (int k = 0; k < KR; ++k) {
        const int n = r + R * k;
#pragma unroll
        for (int c = 0; c < CP; ++c) s[c][k] = (owner && n < N) ? S[(size_t)n * P + p + c] : 0.f;
    }
    const float bias = dt_bias[h], rate = expf(a_log[h]), d_skip = skip[h];
    const bool exact = RT != 0 || R * KR == N;               // no row of a thread lies beyond N

    // one tile's rows into stage `stage`; always one commit, so that groups count tiles
    auto fetch = [&](int t0, int stage) {
        if (t0 < last) {
            const int nt = min(kTile, last - t0);
            const int nv = N / 2, xv = PS / kVec;            // 16-byte pieces of a row of pairs, of a row of x
            for (int v = tid; v < nt * nv; v += blockDim.x) {
                const int tt = v / nv, j = v - tt * nv;      // nv is a constant power of two where RT is set
                copy_async_16(sBC + (stage * kTile + tt) * N + 2 * j, bc + (size_t)(t0 + tt) * ld_bc + g * N + 2 * j);
            }
            for (int v = tid; v < nt * xv; v += blockDim.x) {
                const int tt = v / xv, j = v - tt * xv;
                copy_async_16(rawx + (stage * kTile + tt) * PS + j * kVec, x + (size_t)(t0 + tt) * ld_x + h * P + p0 + j * kVec);
            }
        }
        copy_async_commit();
    };
    if (kAsync) fetch(first, 0);
    float dt_next = 0.f;
    if (tid < kTile && first + tid < last) dt_next = to_f32<T>(dt_raw[(size_t)(first + tid) * ld_dt + h]);

    int stage = 0;
    for (int t0 = first; t0 < last; t0 += kTile, stage ^= 1) {
        const int nt = min(kTile, last - t0);
        __syncthreads();                                     // the tile before has been used up: its stage is free
        if (kAsync) {
            fetch(t0 + kTile, stage ^ 1);
            copy_async_wait_all_but_one();
            __syncthreads();
            for (int idx = tid; idx < nt * PS; idx += blockDim.x) sx[idx] = to_f32<T>(rawx[stage * kTile * PS + idx]);
        } else {
            for (int idx = tid; idx < nt * cols; idx += blockDim.x) {
                const int tt = idx / cols, pp = idx - tt * cols;
                sx[tt * PS + pp] = to_f32<T>(x[(size_t)(t0 + tt) * ld_x + h * P + p0 + pp]);
            }
            for (int idx = tid; idx < nt * N; idx += blockDim.x) {
                const int tt = idx / N, nn = idx - tt * N;
                sBC[(stage * kTile + tt) * N + nn] = bc[(size_t)(t0 + tt) * ld_bc + g * N + nn];
            }
        }
        if (tid < nt) {
            const float dt = softplus_f(dt_next + bias);
            sda[tid] = make_float2(dt, expf(-rate * dt));
        }
        __syncthreads();
        if (tid < kTile && t0 + kTile + tid < last) dt_next = to_f32<T>(dt_raw[(size_t)(t0 + kTile + tid) * ld_dt + h]);
        const float2* tile_bc = sBC + stage * kTile * N + r;
        for (int tq = 0; tq < nt; tq += 4) {
            float acc[4][CP], xs[4][CP];
            if (exact && tq + 4 <= nt) {
                // four whole tokens, no branch in the way: the rows' chains (one per k and column) run
                // side by side, each stepping through the four tokens in order
                float da_a[4], dx[4][CP];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float2 da = sda[tq + u];
                    da_a[u] = da.y;
#pragma unroll
                    for (int c = 0; c < CP; ++c) {
                        xs[u][c] = owner ? sx[(tq + u) * PS + pl + c] : 0.f;
                        dx[u][c] = da.x * xs[u][c];
                        acc[u][c] = 0.f;
                    }
                }
                const float2* row = tile_bc + tq * N;
#pragma unroll
                for (int k = 0; k < KR; ++k) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const float2 v = row[u * N + R * k];
#pragma unroll
                        for (int c = 0; c < CP; ++c) {
                            s[c][k] = fmaf(da_a[u], s[c][k], v.x * dx[u][c]);
                            acc[u][c] = fmaf(s[c][k], v.y, acc[u][c]);
                        }
                    }
                }
            } else {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int tt = tq + u;
#pragma unroll
                    for (int c = 0; c < CP; ++c) { acc[u][c] = 0.f; xs[u][c] = 0.f; }
                    if (tt < nt) {
                        const float2 da = sda[tt];
                        float dx[CP];
#pragma unroll
                        for (int c = 0; c < CP; ++c) {
                            xs[u][c] = owner ? sx[tt * PS + pl + c] : 0.f;
                            dx[c] = da.x * xs[u][c];
                        }
                        const float2* row = tile_bc + tt * N;
#pragma unroll
                        for (int k = 0; k < KR; ++k) {
                            if (r + R * k < N) {
                                const float2 v = row[R * k];
#pragma unroll
                                for (int c = 0; c < CP; ++c) {
                                    s[c][k] = fmaf(da.y, s[c][k], v.x * dx[c]);
                                    acc[u][c] = fmaf(s[c][k], v.y, acc[u][c]);
                                }
                            }
                        }
                    }
                }
            }
            for (int o = R >> 1; o > 0; o >>= 1) {
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int c = 0; c < CP; ++c) acc[u][c] += __shfl_xor_sync(0xffffffffu, acc[u][c], o);
            }
            if (owner && r == 0) {
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (tq + u < nt) {
#pragma unroll
                        for (int c = 0; c < CP; ++c)
                            y[(size_t)(t0 + tq + u) * ld_y + h * P + p + c] = fmaf(d_skip, xs[u][c], acc[u][c]);
                    }
            }
        }
    }
    if (kAsync) asm volatile("cp.async.wait_all;\n" ::: "memory");
    if (owner) {
#pragma unroll
        for (int k = 0; k < KR; ++k) {
            const int n = r + R * k;
            if (n < N) {
#pragma unroll
                for (int c = 0; c < CP; ++c) S[(size_t)n * P + p + c] = s[c][k];
            }
        }
    }
}

// The same recurrence for a step in which every sequence brings one token (row b
// is sequence b's): what costs is reading and writing the state once, so a
// thread owns four neighbouring columns of S (16-byte accesses, a row of S is one
// contiguous run of the block's threads) for the rows n = j, j + J, ...; the J
// partial sums of y meet in shared memory and are added in a fixed order.
template <typename T>
__global__ void ssm_step_kernel(const T* __restrict__ x, int ld_x, const float2* __restrict__ bc, int ld_bc,
                                const T* __restrict__ dt_raw, int ld_dt,
                                const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                const float* __restrict__ skip, float* __restrict__ state,
                                float* __restrict__ y, int ld_y, const int* __restrict__ slots,
                                int heads, int groups, int N, int P, int J) {
    chain_release();
    chain_wait();
    extern __shared__ float smem[];
    float* sB = smem;                 // N
    float* sC = sB + N;               // N
    float* part = sC + N;             // J * P
    const int h = blockIdx.x, b = blockIdx.y;
    const int g = h / (heads / groups);
    const int P4 = P >> 2;
    const int tid = threadIdx.x;
    const T* row = x + (size_t)b * ld_x;
    for (int n = tid; n < N; n += blockDim.x) {
        const float2 v = bc[(size_t)b * ld_bc + g * N + n];
        sB[n] = v.x;
        sC[n] = v.y;
    }
    const int c = tid % P4, j = tid / P4;
    const float dt = softplus_f(to_f32<T>(dt_raw[(size_t)b * ld_dt + h]) + dt_bias[h]);
    const float a = expf(-expf(a_log[h]) * dt);
    float xv[4], dx[4], acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 4; ++i) { xv[i] = to_f32<T>(row[h * P + c * 4 + i]); dx[i] = dt * xv[i]; }
    __syncthreads();
    if (j < J) {
        float4* S = reinterpret_cast<float4*>(state + ((size_t)slots[b] * heads + h) * N * P) + c;
        for (int n = j; n < N; n += J) {
            float4 s = S[(size_t)n * P4];
            const float bn = sB[n], cn = sC[n];
            s.x = fmaf(a, s.x, bn * dx[0]); s.y = fmaf(a, s.y, bn * dx[1]);
            s.z = fmaf(a, s.z, bn * dx[2]); s.w = fmaf(a, s.w, bn * dx[3]);
            acc[0] = fmaf(s.x, cn, acc[0]); acc[1] = fmaf(s.y, cn, acc[1]);
            acc[2] = fmaf(s.z, cn, acc[2]); acc[3] = fmaf(s.w, cn, acc[3]);
            S[(size_t)n * P4] = s;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) part[j * P + c * 4 + i] = acc[i];
    }
    __syncthreads();
    if (tid < P) {
        float sum = 0.f;
        for (int k = 0; k < J; ++k) sum += part[k * P + tid];
        y[(size_t)b * ld_y + h * P + tid] = fmaf(skip[h], to_f32<T>(row[h * P + tid]), sum);
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

// The same for bfloat16 rows where a piece is a multiple of 256 wide: one block per
// row, a thread owns 8 neighbouring channels (16- and 32-byte accesses), a piece is
// a whole number of warps whose sums meet through shared memory in a fixed order.
__global__ void __launch_bounds__(1024)
gated_rmsnorm_bf16_vec_kernel(const float* __restrict__ y, int ld_y, const bf16* __restrict__ z, int ld_z,
                              const float* __restrict__ weight, float eps, bf16* __restrict__ out, int ld_out,
                              int width, int size) {
    chain_release();
    chain_wait();
    __shared__ float warp_ss[32];
    const size_t n = blockIdx.x;
    const int c = threadIdx.x * 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float v[8];
    float ss = 0.f;
    if (c < width) {
        const float4* yp = reinterpret_cast<const float4*>(y + n * ld_y + c);
        const float4 a = yp[0], b = yp[1];
        const uint4 zr = *reinterpret_cast<const uint4*>(z + n * ld_z + c);
        const __nv_bfloat162* zh = reinterpret_cast<const __nv_bfloat162*>(&zr);
        const float yy[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(zh[e]);
            v[2 * e] = yy[2 * e] * silu_f(f.x);
            v[2 * e + 1] = yy[2 * e + 1] * silu_f(f.y);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
    }
    ss = warp_sum(ss);
    if (lane == 0) warp_ss[warp] = ss;
    __syncthreads();
    if (c < width) {
        const int warps_per_piece = size / 256;
        const int w0 = (warp / warps_per_piece) * warps_per_piece;
        float total = 0.f;
        for (int k = 0; k < warps_per_piece; ++k) total += warp_ss[w0 + k];
        const float s = 1.0f / sqrtf(total / (float)size + eps);
        const float4* wp = reinterpret_cast<const float4*>(weight + c);
        const float4 w0v = wp[0], w1v = wp[1];
        const float w[8] = {w0v.x, w0v.y, w0v.z, w0v.w, w1v.x, w1v.y, w1v.z, w1v.w};
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(v[2 * e] * s * w[2 * e], v[2 * e + 1] * s * w[2 * e + 1]);
        *reinterpret_cast<uint4*>(out + n * ld_out + c) = o;
    }
}

}  // namespace

GTG_API int gtg_causal_conv_silu(int dtype, const void* in, int ld_in, const float* w, const float* bias,
                                 const float* conv_state, void* out, int ld_out, const int* token_seq,
                                 const int* cu_seqlens, const int* slots, int n_tokens, int C, int taps,
                                 int n_plain, float* pairs, cudaStream_t stream) {
    if (n_tokens <= 0 || C <= 0) return 0;
    if (pairs == nullptr) n_plain = C;
    if (taps < 1 || ld_in < C || ld_out < n_plain || (taps > 1 && conv_state == nullptr)) return kErrBadArgument;
    if (n_plain < 0 || n_plain > C || (C - n_plain) % 2) return kErrBadArgument;
    if ((C + 127) / 128 > 65535) return kErrUnsupported;
    if (dtype == 1 && C % 8 == 0 && ld_in % 8 == 0 && ld_out % 8 == 0 && ((uintptr_t)in % 16) == 0 &&
        ((uintptr_t)out % 16) == 0 && ((uintptr_t)conv_state % 16) == 0 && ((uintptr_t)w % 16) == 0 &&
        n_plain % 8 == 0 && (C - n_plain) % 16 == 0) {
        const int per_block = C / 8 < 128 ? (C / 8 + 31) / 32 * 32 : 128;
        if (n_tokens >= 4 * kConvRun && taps >= 2 && taps <= 4) {            // a prompt: runs of tokens per thread
            const dim3 grid_run((n_tokens + kConvRun - 1) / kConvRun, (C / 8 + per_block - 1) / per_block);
#define GTG_CONV_RUN(TAPS) launch_chained(causal_conv_silu_bf16_run_kernel<TAPS>, grid_run, dim3(per_block), 0, stream, (const bf16*)in, ld_in, w, bias, conv_state, (bf16*)out, ld_out, token_seq, cu_seqlens, slots, n_tokens, C, n_plain, pairs)
            if (taps == 2) return GTG_CONV_RUN(2);
            if (taps == 3) return GTG_CONV_RUN(3);
            return GTG_CONV_RUN(4);
#undef GTG_CONV_RUN
        }
        const dim3 grid_vec(n_tokens, (C / 8 + per_block - 1) / per_block);
        return launch_chained(causal_conv_silu_bf16_vec_kernel, grid_vec, dim3(per_block), 0, stream, (const bf16*)in, ld_in, w, bias, conv_state, (bf16*)out, ld_out, token_seq, cu_seqlens, slots, C, taps, n_plain, pairs);
    }
    const dim3 grid(n_tokens, (C + 127) / 128);
    if (dtype == 0) return launch_chained(causal_conv_silu_kernel<float>, grid, dim3(128), 0, stream, (const float*)in, ld_in, w, bias, conv_state, (float*)out, ld_out, token_seq, cu_seqlens, slots, C, taps, n_plain, pairs);
    if (dtype == 1) return launch_chained(causal_conv_silu_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)in, ld_in, w, bias, conv_state, (bf16*)out, ld_out, token_seq, cu_seqlens, slots, C, taps, n_plain, pairs);
    return kErrBadArgument;
}

GTG_API int gtg_causal_conv_step(int dtype, const void* in, int ld_in, const float* w, const float* bias,
                                 float* conv_state, void* out, int ld_out, const int* slots, int n_seqs, int C,
                                 int taps, int n_plain, float* pairs, cudaStream_t stream) {
    if (n_seqs <= 0 || C <= 0) return 0;
    if (pairs == nullptr) n_plain = C;
    if (taps < 1 || ld_in < C || ld_out < n_plain || (taps > 1 && conv_state == nullptr)) return kErrBadArgument;
    if (n_plain < 0 || n_plain > C || (C - n_plain) % 2) return kErrBadArgument;
    if ((C + 127) / 128 > 65535) return kErrUnsupported;
    const dim3 grid(n_seqs, (C + 127) / 128);
    if (dtype == 0) return launch_chained(causal_conv_step_kernel<float>, grid, dim3(128), 0, stream, (const float*)in, ld_in, w, bias, conv_state, (float*)out, ld_out, slots, C, taps, n_plain, pairs);
    if (dtype == 1) return launch_chained(causal_conv_step_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)in, ld_in, w, bias, conv_state, (bf16*)out, ld_out, slots, C, taps, n_plain, pairs);
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
// leaves a thread at most kRowsPerThread rows (few threads per column mean few
// shuffle rounds per token), but a warp's worth of threads in the block at least.
static int scan_split(int N, int cols) {
    int R = 1;
    while (R < 32 && (N + R - 1) / R > kRowsPerThread) R *= 2;
    while (R < 32 && R * 2 <= N && cols * R < 32) R *= 2;
    return R;
}

GTG_API int gtg_ssm_scan(int dtype, const void* x, int ld_x, const float* bc, int ld_bc, const void* dt_raw, int ld_dt,
                         const float* dt_bias, const float* a_log, const float* skip, float* state,
                         float* y, int ld_y, const int* cu_seqlens, const int* slots, int n_seqs,
                         int heads, int groups, int N, int P, int one_token_each, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (heads <= 0 || groups <= 0 || heads % groups || N <= 0 || P <= 0) return kErrBadArgument;
    if (ld_x < heads * P || ld_bc < groups * N || ((uintptr_t)bc % 8)) return kErrBadArgument;
    if (n_seqs > 65535) return kErrUnsupported;
    const float2* pairs = (const float2*)bc;
    if (one_token_each && P % 4 == 0 && P <= 1024 && ((uintptr_t)state % 16) == 0) {
        const int P4 = P / 4;
        int J = 256 / P4;
        if (J < 1) J = 1;
        if (J > N) J = N;
        int threads = (P4 * J + 31) / 32 * 32;
        if (threads < P) threads = (P + 31) / 32 * 32;
        const size_t smem_step = (size_t)(2 * N + J * P) * sizeof(float);
        if (threads <= 1024 && smem_step <= 48 * 1024) {
            const dim3 grid_step(heads, n_seqs);
            if (dtype == 0) return launch_chained(ssm_step_kernel<float>, grid_step, dim3(threads), smem_step, stream, (const float*)x, ld_x, pairs, ld_bc, (const float*)dt_raw, ld_dt, dt_bias, a_log, skip, state, y, ld_y, slots, heads, groups, N, P, J);
            if (dtype == 1) return launch_chained(ssm_step_kernel<bf16>, grid_step, dim3(threads), smem_step, stream, (const bf16*)x, ld_x, pairs, ld_bc, (const bf16*)dt_raw, ld_dt, dt_bias, a_log, skip, state, y, ld_y, slots, heads, groups, N, P, J);
            return kErrBadArgument;
        }
    }
    static int n_sm = 0;
    if (n_sm == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0)
            n_sm = 148;
    }
    // Slices of columns, so that a few long sequences still give a block to most
    // multiprocessors (measured at 64 heads of 64 columns and a state of 128: two slices
    // of 32 columns, 128 blocks, 0.46 ms for 2,048 tokens; four slices 0.49, eight 0.55:
    // every slice stages the head's B and C again).  Where every run of x and of the pairs starts on a 16-byte boundary
    // the slices are halves, quarters, ... of a head that keep that alignment and the rows
    // come by asynchronous copies; otherwise slices of at least four columns, read plainly.
    const int vec = dtype == 0 ? 4 : 8;
    const bool aligned = N % 2 == 0 && ld_bc % 2 == 0 && ((uintptr_t)bc % 16) == 0 &&
                         P % vec == 0 && ld_x % vec == 0 && ((uintptr_t)x % 16) == 0;
    int PS = P;
    if (aligned) {
        while (2LL * heads * n_seqs * (P / PS) <= (long long)n_sm && PS % 2 == 0 && (PS / 2) % vec == 0) PS /= 2;
    } else {
        int slices = (n_sm + heads * n_seqs - 1) / (heads * n_seqs);
        if (slices > (P + 3) / 4) slices = (P + 3) / 4;
        if (slices < 1) slices = 1;
        PS = (P + slices - 1) / slices;
    }
    const int slices = (P + PS - 1) / PS;
    int R = scan_split(N, PS);
    if ((N + R - 1) / R > kRowsPerThread) return kErrUnsupported;
    const int threads = (PS * R + 31) / 32 * 32;
    if (threads > 1024) return kErrUnsupported;
    const bool constants = aligned && N == R * 16 && (R == 2 || R == 4 || R == 8 || R == 16);   // R and N known to the kernel
    const int kTile = constants ? kMaxTile : kPlainTile;
    size_t smem = (size_t)(4 * kTile * N + kTile * PS + 1 + 2 * kTile) * sizeof(float);
    if (aligned) smem += (size_t)2 * kTile * PS * (dtype == 0 ? 4 : 2);
    if (smem > 200 * 1024) return kErrUnsupported;
    const dim3 grid(heads, n_seqs, slices);
    cudaError_t e;
    const int rows = (N + R - 1) / R;
#define GTG_SCAN_LAUNCH_KR(T, ASYNC, KR, RT, CP)                                                                         \
    do {                                                                                                                 \
        if (smem > 48 * 1024 && (e = cudaFuncSetAttribute(ssm_scan_kernel<T, ASYNC, KR, RT, CP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)e; \
        return launch_chained(ssm_scan_kernel<T, ASYNC, KR, RT, CP>, grid, dim3(((PS / CP) * R + 31) / 32 * 32), smem, stream, (const T*)x, ld_x, pairs, ld_bc, (const T*)dt_raw, ld_dt, dt_bias, a_log, skip, state, y, ld_y, cu_seqlens, slots, heads, groups, N, P, R, PS); \
    } while (0)
#define GTG_SCAN_LAUNCH(T, ASYNC)                                                                                        \
    do {                                                                                                                 \
        if (ASYNC && constants) {                /* the usual state sizes: R and N constants of the kernel */            \
            if (R == 2) GTG_SCAN_LAUNCH_KR(T, ASYNC, 16, 2, 2);                                                          \
            if (R == 4) GTG_SCAN_LAUNCH_KR(T, ASYNC, 16, 4, 2);                                                          \
            if (R == 8) GTG_SCAN_LAUNCH_KR(T, ASYNC, 16, 8, 2);                                                          \
            if (R == 16) GTG_SCAN_LAUNCH_KR(T, ASYNC, 16, 16, 2);                                                        \
        }                                                                                                                \
        if (rows <= 4) GTG_SCAN_LAUNCH_KR(T, ASYNC, 4, 0, 1);                                                            \
        if (rows <= 8) GTG_SCAN_LAUNCH_KR(T, ASYNC, 8, 0, 1);                                                            \
        GTG_SCAN_LAUNCH_KR(T, ASYNC, 16, 0, 1);                                                                          \
    } while (0)
    if (dtype == 0) { if (aligned) GTG_SCAN_LAUNCH(float, true); else GTG_SCAN_LAUNCH(float, false); }
    if (dtype == 1) { if (aligned) GTG_SCAN_LAUNCH(bf16, true); else GTG_SCAN_LAUNCH(bf16, false); }
#undef GTG_SCAN_LAUNCH_KR
#undef GTG_SCAN_LAUNCH
    return kErrBadArgument;
}

GTG_API int gtg_gated_rmsnorm(int dtype, const float* y, int ld_y, const void* z, int ld_z, const float* weight,
                              float eps, void* out, int ld_out, int n_rows, int width, int parts,
                              cudaStream_t stream) {
    if (n_rows <= 0 || width <= 0) return 0;
    if (parts <= 0 || width % parts || parts > 65535) return kErrBadArgument;
    const int size = width / parts;
    if (dtype == 1 && size % 256 == 0 && width <= 8192 && ld_y % 4 == 0 && ld_z % 8 == 0 && ld_out % 8 == 0 &&
        ((uintptr_t)y % 16) == 0 && ((uintptr_t)z % 16) == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)weight % 16) == 0)
        return launch_chained(gated_rmsnorm_bf16_vec_kernel, dim3(n_rows), dim3(width / 8), 0, stream, y, ld_y, (const bf16*)z, ld_z, weight, eps, (bf16*)out, ld_out, width, size);
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
