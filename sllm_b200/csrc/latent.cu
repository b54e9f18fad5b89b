// Kernels of latent attention: every head's keys and values are up-projections of one small latent
// vector per token, and only that vector is cached.
//
//   * latent_write: the latent of each new token (columns of a float32 product) over its root mean square,
//     times a gain, written to the token's place in the paged cache in the cache's dtype.
//   * head_linear: a product per head, out[t, h, :] = W_h x[t, h, :], with W [H, dout, din].  It carries a
//     head's query into the latent space (W_h = the head's key up-projection, transposed: the score of a
//     query against a key is then its carried form against the cached latent) and the head's weighted sum
//     of latents back out through the value up-projection; there the result can be multiplied by
//     sigmoid(gate[t, h]) as it is written.  float32 accumulation over din in a fixed order.
#include "common.cuh"

namespace sllm {

template <typename TC>
__global__ void latent_write_kernel(const float* __restrict__ proj, int ld, int off, int rank, const float* __restrict__ gain,
                                    float eps, const int* __restrict__ slot_mapping, TC* __restrict__ cache) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int slot = slot_mapping[t];
  const float* x = proj + (size_t)t * ld + off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
  const float total = block_sum(ss, red);
  if (slot < 0) return;               // a row that pads the batch: no place to write to
  const float inv = 1.0f / sqrtf(total / (float)rank + eps);
  TC* dst = cache + (size_t)slot * rank;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f32<TC>(x[i] * inv * gain[i]);
}

constexpr int HL_BM = 64, HL_BN = 64, HL_BK = 16;

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
head_linear_kernel(const TX* __restrict__ x, int ldx, int xoff, const TW* __restrict__ w, TO* __restrict__ out,
                   const float* __restrict__ gate, int ldg, int goff, int T, int H, int din, int dout) {
  __shared__ float Xs[HL_BK][HL_BM + 4];
  __shared__ float Ws[HL_BK][HL_BN + 4];
  pdl_wait();
  const int h = blockIdx.z;
  const int m0 = blockIdx.y * HL_BM, n0 = blockIdx.x * HL_BN;
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int lr = tid / 4, lk = (tid % 4) * 4;
  const TX* xh = x + xoff + (size_t)h * din;
  const TW* wh = w + (size_t)h * dout * din;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < din; k0 += HL_BK) {
    float a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int gk = k0 + lk + i;
      a[i] = (m0 + lr < T && gk < din) ? to_f32(xh[(size_t)(m0 + lr) * ldx + gk]) : 0.f;
      b[i] = (n0 + lr < dout && gk < din) ? to_f32(wh[(size_t)(n0 + lr) * din + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) { Xs[lk + i][lr] = a[i]; Ws[lk + i][lr] = b[i]; }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < HL_BK; ++k) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = Xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
  }
  pdl_launch_dependents();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= T) continue;
    const float g = gate != nullptr ? 1.0f / (1.0f + expf(-gate[(size_t)m * ldg + goff + h])) : 1.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < dout) out[(size_t)m * H * dout + (size_t)h * dout + n] = from_f32<TO>(acc[i][j] * g);
    }
  }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_latent_write(const float* proj, int ld, int off, int rank, const float* gain, float eps,
                                  const int* slot_mapping, void* cache, int cache_dtype, int T, cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && rank > 0 && off >= 0 && off + rank <= ld, "latent_write: columns %d..%d of %d", off, off + rank, ld);
  if (T == 0) return SLLM_OK;
  const int threads = rank >= 512 ? 256 : 128;
  if (cache_dtype == SLLM_F32)
    launch_kernel(latent_write_kernel<float>, T, threads, 0, stream, proj, ld, off, rank, gain, eps, slot_mapping, (float*)cache);
  else if (cache_dtype == SLLM_BF16)
    launch_kernel(latent_write_kernel<__nv_bfloat16>, T, threads, 0, stream, proj, ld, off, rank, gain, eps, slot_mapping,
                  (__nv_bfloat16*)cache);
  else
    SLLM_REQUIRE(false, "latent_write: unknown dtype %d", cache_dtype);
  return launch_status("latent_write");
}

SLLM_EXPORT int sllm_head_linear(const void* x, int x_dtype, int ldx, int xoff, const void* w, int w_dtype, void* out, int out_dtype,
                                 const float* gate, int ldg, int goff, int T, int H, int din, int dout, cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && H > 0 && H <= 65535 && din > 0 && dout > 0, "head_linear: bad sizes T=%d H=%d din=%d dout=%d", T, H, din, dout);
  SLLM_REQUIRE(xoff >= 0 && xoff + H * din <= ldx, "head_linear: columns %d..%d of %d", xoff, xoff + H * din, ldx);
  SLLM_REQUIRE(gate == nullptr || (goff >= 0 && goff + H <= ldg), "head_linear: gate columns outside %d", ldg);
  if (T == 0) return SLLM_OK;
  const dim3 grid((unsigned)((dout + HL_BN - 1) / HL_BN), (unsigned)((T + HL_BM - 1) / HL_BM), (unsigned)H);
  SLLM_REQUIRE(grid.y <= 65535, "head_linear: too many rows for one launch");
#define SLLM_HL(TX, TW, TO)                                                                                              \
  launch_kernel(head_linear_kernel<TX, TW, TO>, grid, 256, 0, stream, (const TX*)x, ldx, xoff, (const TW*)w, (TO*)out, gate, ldg, \
                goff, T, H, din, dout)
  if (x_dtype == SLLM_F32 && w_dtype == SLLM_F32 && out_dtype == SLLM_F32) SLLM_HL(float, float, float);
  else if (x_dtype == SLLM_F32 && w_dtype == SLLM_BF16 && out_dtype == SLLM_BF16) SLLM_HL(float, __nv_bfloat16, __nv_bfloat16);
  else if (x_dtype == SLLM_BF16 && w_dtype == SLLM_BF16 && out_dtype == SLLM_BF16) SLLM_HL(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  else SLLM_REQUIRE(false, "head_linear: dtypes x=%d w=%d out=%d", x_dtype, w_dtype, out_dtype);
#undef SLLM_HL
  return launch_status("head_linear");
}
