// A mixture of experts' router and the activation that carries its weights.
//
//   moe_route   per token, from float32 router logits z [T, E]: s = sigmoid(z); choice = s + correction; the experts
//               form `groups` equal groups of neighbours, a group's score is the sum of its two largest choice scores
//               (its only one, for groups of one), only experts of the `keep` best groups can be chosen; the `top`
//               largest choice scores among them win (the lower index on a tie); a winner's weight is s * scale, not
//               renormalized.  Written as a dense float32 row [E] with zeros for the others, and as (index, weight) lists.
//   moe_act     act[t, c] = gelu(up[t, c]) * weight[t, c / ff] for the routed experts' columns (all experts' up
//               projections are ONE matrix, expert e's rows at e * ff), and gelu(up) alone for the columns of the
//               expert every token uses that follow them; gelu in its exact (erf) form, float32.
//               The down projections, side by side as one matrix, then add up the weighted experts by themselves.
#include <math.h>

#include "common.cuh"

namespace sllm {

constexpr int ROUTE_WARPS = 4;

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ correction, int T, int E, int groups, int keep,
                 int top, float scale, float* __restrict__ dense, int* __restrict__ idx, float* __restrict__ wts) {
  extern __shared__ float sm[];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= T) return;
  float* choice = sm + (size_t)warp * (E + groups);
  float* gscore = choice + E;
  const float* z = logits + (size_t)t * E;
  for (int e = lane; e < E; e += 32) {
    choice[e] = 1.0f / (1.0f + expf(-z[e])) + (correction ? correction[e] : 0.f);
    dense[(size_t)t * E + e] = 0.f;
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int per = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;          // the two largest
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float c = choice[e];
        if (c > a) { b = a; a = c; } else if (c > b) { b = c; }
      }
      gscore[g] = per > 1 ? a + b : a;
    }
    __syncwarp();
    // the groups that stay: the keep best, marked by +inf; then every other group's experts leave
    for (int n = 0; n < keep; ++n) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        const float v = gscore[g];
        if (v != INFINITY && (v > bv || (v == bv && g < bi))) { bv = v; bi = g; }
      }
      warp_argmax(bv, bi);
      if (lane == 0 && bi < groups) gscore[bi] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gscore[e / per] != INFINITY) choice[e] = -INFINITY;
    __syncwarp();
  }
  for (int n = 0; n < top; ++n) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = choice[e];
      if (!isnan(v) && (v > bv || (v == bv && e < bi))) { bv = v; bi = e; }
    }
    warp_argmax(bv, bi);
    if (lane == 0) {
      float w = 0.f;
      int e = bi < E ? bi : 0;
      if (bi < E && bv != -INFINITY) {
        w = scale / (1.0f + expf(-z[e]));
        dense[(size_t)t * E + e] = w;
        choice[e] = NAN;                            // taken
      }
      idx[(size_t)t * top + n] = e;
      wts[(size_t)t * top + n] = w;
    }
    __syncwarp();
  }
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
moe_act_kernel(const TI* __restrict__ up, const float* __restrict__ dense, TO* __restrict__ out, int N, int E, int ff) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int routed = E * ff;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < N; c += gridDim.y * blockDim.x) {
    const float w = c < routed ? dense[(size_t)t * E + c / ff] : 1.f;
    float y = 0.f;
    if (w != 0.f) {
      const float z = to_f32(up[(size_t)t * N + c]);
      y = 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f)) * w;
    }
    out[(size_t)t * N + c] = from_f32<TO>(y);
  }
}

// The same for bfloat16 in and out, eight columns a thread (one 16-byte load and store): needs ff, N and the routed
// experts' columns to be multiples of 8, so that a thread's columns share one expert.  The columns of an expert that a
// token does not use are not read.
__global__ void __launch_bounds__(256)
moe_act_vec_kernel(const __nv_bfloat16* __restrict__ up, const float* __restrict__ dense, __nv_bfloat16* __restrict__ out, int N,
                   int E, int ff) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int routed = E * ff;
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8; c < N; c += gridDim.y * blockDim.x * 8) {
    const float w = c < routed ? dense[(size_t)t * E + c / ff] : 1.f;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (w != 0.f) {
      raw = *reinterpret_cast<const uint4*>(up + (size_t)t * N + c);
      __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 z = __bfloat1622float2(h2[k]);
        z.x = 0.5f * z.x * (1.0f + erff(z.x * 0.70710678118654752440f)) * w;
        z.y = 0.5f * z.y * (1.0f + erff(z.y * 0.70710678118654752440f)) * w;
        h2[k] = __floats2bfloat162_rn(z.x, z.y);
      }
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * N + c) = raw;
  }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_moe_route(const float* logits, const float* correction, int T, int E, int groups, int keep, int top,
                               float scale, float* dense, int* idx, float* wts, cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && E >= 1 && top >= 1 && top <= E, "moe_route: bad sizes T=%d E=%d top=%d", T, E, top);
  SLLM_REQUIRE(groups >= 1 && E % groups == 0 && keep >= 1 && keep <= groups, "moe_route: %d groups (keep %d) of %d experts", groups, keep, E);
  SLLM_REQUIRE((long)keep * (E / groups) >= top, "moe_route: %d groups of %d experts cannot give %d", keep, E / groups, top);
  const size_t smem = (size_t)ROUTE_WARPS * (E + groups) * sizeof(float);
  SLLM_REQUIRE(smem <= 48 * 1024, "moe_route: %d experts are more than the kernel keeps in shared memory", E);
  if (T == 0) return SLLM_OK;
  launch_kernel(moe_route_kernel, (unsigned)((T + ROUTE_WARPS - 1) / ROUTE_WARPS), ROUTE_WARPS * 32, smem, stream, logits,
                correction, T, E, groups, keep, top, scale, dense, idx, wts);
  return launch_status("moe_route");
}

SLLM_EXPORT int sllm_moe_act(const void* up, int in_dtype, const float* dense, void* out, int out_dtype, int T, int N, int E, int ff,
                             cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && N >= 1 && E >= 0 && ff >= 1 && (long)E * ff <= N, "moe_act: bad sizes T=%d N=%d E=%d ff=%d", T, N, E, ff);
  if (T == 0) return SLLM_OK;
  if (in_dtype == SLLM_BF16 && out_dtype == SLLM_BF16 && N % 8 == 0 && ff % 8 == 0 && (uintptr_t)up % 16 == 0 &&
      (uintptr_t)out % 16 == 0) {
    int by = (N / 8 + 255) / 256;
    if (by > 64) by = 64;
    launch_kernel(moe_act_vec_kernel, dim3((unsigned)T, (unsigned)by), 256, 0, stream, (const __nv_bfloat16*)up, dense,
                  (__nv_bfloat16*)out, N, E, ff);
    return launch_status("moe_act");
  }
  int by = (N + 255) / 256;
  if (by > 64) by = 64;
  const dim3 grid((unsigned)T, (unsigned)by);
#define LAUNCH(TI, TO) launch_kernel(moe_act_kernel<TI, TO>, grid, 256, 0, stream, (const TI*)up, dense, (TO*)out, N, E, ff)
  if (in_dtype == SLLM_F32 && out_dtype == SLLM_F32) LAUNCH(float, float);
  else if (in_dtype == SLLM_F32 && out_dtype == SLLM_BF16) LAUNCH(float, __nv_bfloat16);
  else if (in_dtype == SLLM_BF16 && out_dtype == SLLM_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else SLLM_REQUIRE(false, "moe_act: unsupported dtypes %d -> %d", in_dtype, out_dtype);
#undef LAUNCH
  return launch_status("moe_act");
}
