// Attention through a latent: what stands between the projections and the
// attention kernel.
//
// A token leaves two things in the cache instead of keys and values per head: a
// latent vector c of `rank` channels, normed (c = x / sqrt(mean(x^2) + eps) * w
// over the rank channels of the down projection), and one rotated key part of
// `rot` channels that all heads share.  A cache row is [c | rotated part]:
// rank + rot channels of a single key/value head.  Head h's unrotated key would
// be U_h c; its score against a query q_h = [a_h | b_h] is
//     a_h . (U_h c) + b_h' . k'  =  (U_h^T a_h) . c + b_h' . k'        (' = rotated)
// so the query that meets the cache row is [U_h^T a_h | b_h'], also rank + rot
// channels, and the value of a row is its first rank channels.
//
// latent_prepare, one block per token, does the per-token work in float:
//   * with a down projection: the norm of the latent, the rotation of the shared
//     key part, and the store of both into the token's cache row;
//   * the rotation of every head's b_h into the tail of the head's query row
//     (the head of the row is written by the product with U_h^T).
// Rotation: of the part's first `rdims` channels, (2i, 2i+1) turn by the angle of pair i, whose cosine and
// sine (amplitude included) come from the step's table [token, rot/2].
#include "common.cuh"
#include <math.h>

namespace {
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ dkv, int ldd,
                      const float2* __restrict__ cos_sin, const float* __restrict__ norm_w, float eps,
                      T* __restrict__ kc, long long page_stride, const int* __restrict__ block_table,
                      int table_stride, const int* __restrict__ token_seq, const int* __restrict__ slots,
                      const int* __restrict__ positions, T* __restrict__ q_full, int ldf,
                      int n_heads, int dim, int rot, int rdims, int rank) {
    chain_release();
    chain_wait();
    __shared__ float scratch[33];
    const int n = blockIdx.x;
    const int half = rdims / 2;   // pairs that turn; channels rdims..rot-1 of the part pass unchanged
    const float2* cs = cos_sin + (size_t)n * half;
    if (dkv) {
        const T* d = dkv + (size_t)n * ldd;
        float ss = 0.f;
        for (int i = threadIdx.x; i < rank; i += blockDim.x) {
            const float x = to_f32<T>(d[i]);
            ss += x * x;
        }
        const float total = block_sum(ss, scratch);
        const float s = 1.0f / sqrtf(total / (float)rank + eps);
        const int pos = positions[n];
        const int slot = slots[token_seq[n]];
        const int page = block_table[(size_t)slot * table_stride + pos / kPageTokens];
        T* row = kc + (size_t)page * page_stride + (size_t)(pos % kPageTokens) * (rank + rot);
        for (int i = threadIdx.x; i < rank; i += blockDim.x)
            row[i] = from_f32<T>((norm_w[i] * to_f32<T>(d[i])) * s);
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float u = to_f32<T>(d[rank + 2 * i]), v = to_f32<T>(d[rank + 2 * i + 1]);
            const float2 a = cs[i];
            row[rank + 2 * i] = from_f32<T>(u * a.x - v * a.y);
            row[rank + 2 * i + 1] = from_f32<T>(v * a.x + u * a.y);
        }
        for (int i = rdims + threadIdx.x; i < rot; i += blockDim.x) row[rank + i] = d[rank + i];
    }
    const int D = rank + rot;
    for (int idx = threadIdx.x; idx < n_heads * half; idx += blockDim.x) {
        const int h = idx / half, i = idx % half;
        const T* src = q + (size_t)n * ldq + (size_t)h * (dim + rot) + dim;
        const float u = to_f32<T>(src[2 * i]), v = to_f32<T>(src[2 * i + 1]);
        const float2 a = cs[i];
        T* dst = q_full + (size_t)n * ldf + (size_t)h * D + rank;
        dst[2 * i] = from_f32<T>(u * a.x - v * a.y);
        dst[2 * i + 1] = from_f32<T>(v * a.x + u * a.y);
    }
    for (int idx = threadIdx.x; idx < n_heads * (rot - rdims); idx += blockDim.x) {
        const int h = idx / (rot - rdims), i = rdims + idx % (rot - rdims);
        q_full[(size_t)n * ldf + (size_t)h * D + rank + i] = q[(size_t)n * ldq + (size_t)h * (dim + rot) + dim + i];
    }
}
}  // namespace

GTG_API int gtg_latent_prepare(int dtype, const void* q, int ldq, const void* dkv, int ldd, const float* cos_sin,
                               const float* norm_w, float eps, void* kc, long long page_stride,
                               const int* block_table, int table_stride, const int* token_seq, const int* slots,
                               const int* positions, void* q_full, int ldf, int N, int n_heads, int dim, int rot,
                               int rdims, int rank, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_heads <= 0 || dim <= 0 || rot <= 0 || rdims < 0 || rdims > rot || rdims % 2 || rank <= 0) return kErrBadArgument;
    if (dkv && (!kc || !norm_w || !block_table)) return kErrBadArgument;
    if (dtype == 0)
        return launch_chained(latent_prepare_kernel<float>, dim3(N), dim3(128), 0, stream, (const float*)q, ldq,
                              (const float*)dkv, ldd, (const float2*)cos_sin, norm_w, eps, (float*)kc, page_stride,
                              block_table, table_stride, token_seq, slots, positions, (float*)q_full, ldf, n_heads,
                              dim, rot, rdims, rank);
    if (dtype == 1)
        return launch_chained(latent_prepare_kernel<bf16>, dim3(N), dim3(128), 0, stream, (const bf16*)q, ldq,
                              (const bf16*)dkv, ldd, (const float2*)cos_sin, norm_w, eps, (bf16*)kc, page_stride,
                              block_table, table_stride, token_seq, slots, positions, (bf16*)q_full, ldf, n_heads,
                              dim, rot, rdims, rank);
    return kErrBadArgument;
}
