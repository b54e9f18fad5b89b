// The generalized delta rule: a recurrent mixer with a float32 matrix state S [dk, dv] per request and head.
//
//   S <- diag(d) S - (a * u) (u^T S) + k v^T        (S on the right is the state before the token)
//   o  = S^T r
//
// d = exp(-exp(-1/2) * sigmoid(decay logit)) per key channel, a = sigmoid(removal logit + bias) per key
// channel, u = k / sqrt(sum(k^2) + 1e-6) per head.  Everything that enters the recurrence is float32: the
// projections arrive as float32 columns of one product, the decays, rates, unit keys, the state and the
// outputs are float32.
//
// The columns of S evolve independently of one another (column j needs u, d, a*u, k, r of the token and
// v_j only), so a CTA owns a slice of DR_COLS columns of one (request, head) and walks the request's tokens
// in order.  Four consecutive lanes share a column, each holding every fourth row in registers; the two
// sums over rows of a step are two shuffles each.  The token's vectors are prepared for DR_CHUNK tokens at a
// time in shared memory (one CTA-wide barrier pair per chunk, none per token).  A portion of a prompt and
// a single decoded token run through the same kernel, from the state slot and back into it.
//
// A second kernel finishes the mixer's output: each head's o over its root mean square, times a gain,
// times sigmoid(gate logit), in the compute dtype.
#include "common.cuh"

namespace sllm {

constexpr int DR_COLS = 32;      // columns of S per CTA
constexpr int DR_SPLIT = 4;      // lanes per column
constexpr int DR_THREADS = DR_COLS * DR_SPLIT;
constexpr int DR_MAX_CHUNK = 16;

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

struct DeltaParams {
  const float* proj;       // [T, ld]: columns off_r, off_k (+ h*dk), off_v (+ h*dv), off_a (+ h*dk)
  const float* decay;      // [T, H*dk] decay logits
  const float* a_bias;     // [H*dk]
  float* state;            // [slots, H, dk, dv]
  const int* q_start;      // [S+1]
  const int* state_slots;  // [S]
  float* out;              // [T, H*dv]
  int ld, off_r, off_k, off_v, off_a, H, dk, dv, chunk;
};

// RPT: rows of a column per lane (dk <= 4 * RPT).
template <int RPT>
__global__ void __launch_bounds__(DR_THREADS) delta_rule_kernel(const DeltaParams p) {
  extern __shared__ float sm[];
  const int dk = p.dk, dv = p.dv, chunk = p.chunk;
  float* s_u = sm;                        // [chunk][dk] unit key
  float* s_d = s_u + chunk * dk;          // decay
  float* s_au = s_d + chunk * dk;         // removal rate * unit key
  float* s_k = s_au + chunk * dk;
  float* s_r = s_k + chunk * dk;
  float* s_v = s_r + chunk * dk;          // [chunk][DR_COLS]
  float* s_ss = s_v + chunk * DR_COLS;    // [chunk] sum of k^2
  pdl_wait();
  const int seq = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * DR_COLS;
  const int t_begin = p.q_start[seq], t_end = p.q_start[seq + 1];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int col = c0 + tid / DR_SPLIT, rs = tid % DR_SPLIT;
  const bool live = col < dv;
  float* S = p.state + ((size_t)p.state_slots[seq] * p.H + h) * dk * dv;
  float s[RPT];
#pragma unroll
  for (int n = 0; n < RPT; ++n) {
    const int i = n * DR_SPLIT + rs;
    s[n] = (live && i < dk) ? S[(size_t)i * dv + col] : 0.f;
  }
  const float c_decay = -expf(-0.5f);
  for (int t0 = t_begin; t0 < t_end; t0 += chunk) {
    const int nt = min(chunk, t_end - t0);
    __syncthreads();                       // the chunk before has been read
    // sum of squares of each token's key: a warp per token
    for (int tt = warp; tt < nt; tt += DR_THREADS / 32) {
      const float* k = p.proj + (size_t)(t0 + tt) * p.ld + p.off_k + h * dk;
      float ss = 0.f;
      for (int i = lane; i < dk; i += 32) ss = fmaf(k[i], k[i], ss);
      ss = warp_sum(ss);
      if (lane == 0) s_ss[tt] = ss;
    }
    __syncthreads();
    for (int e = tid; e < nt * dk; e += DR_THREADS) {
      const int tt = e / dk, i = e % dk;
      const float* row = p.proj + (size_t)(t0 + tt) * p.ld;
      const float k = row[p.off_k + h * dk + i];
      const float u = k / sqrtf(s_ss[tt] + 1e-6f);
      const float a = sigmoidf_(row[p.off_a + h * dk + i] + p.a_bias[h * dk + i]);
      s_k[e] = k;
      s_u[e] = u;
      s_au[e] = a * u;
      s_d[e] = expf(c_decay * sigmoidf_(p.decay[(size_t)(t0 + tt) * p.H * dk + h * dk + i]));
      s_r[e] = row[p.off_r + h * dk + i];
    }
    for (int e = tid; e < nt * DR_COLS; e += DR_THREADS) {
      const int tt = e / DR_COLS, j = c0 + e % DR_COLS;
      s_v[e] = j < dv ? p.proj[(size_t)(t0 + tt) * p.ld + p.off_v + h * dv + j] : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float* u = s_u + tt * dk;
      const float* d = s_d + tt * dk;
      const float* au = s_au + tt * dk;
      const float* k = s_k + tt * dk;
      const float* r = s_r + tt * dk;
      float us = 0.f;
#pragma unroll
      for (int n = 0; n < RPT; ++n) {
        const int i = n * DR_SPLIT + rs;
        if (i < dk) us = fmaf(u[i], s[n], us);
      }
      us += __shfl_xor_sync(0xffffffffu, us, 1);
      us += __shfl_xor_sync(0xffffffffu, us, 2);
      const float v = s_v[tt * DR_COLS + tid / DR_SPLIT];
      float o = 0.f;
#pragma unroll
      for (int n = 0; n < RPT; ++n) {
        const int i = n * DR_SPLIT + rs;
        if (i < dk) {
          s[n] = fmaf(k[i], v, fmaf(-au[i], us, d[i] * s[n]));
          o = fmaf(s[n], r[i], o);
        }
      }
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (live && rs == 0) p.out[(size_t)(t0 + tt) * p.H * dv + h * dv + col] = o;
    }
  }
  pdl_launch_dependents();
  if (live) {
#pragma unroll
    for (int n = 0; n < RPT; ++n) {
      const int i = n * DR_SPLIT + rs;
      if (i < dk) S[(size_t)i * dv + col] = s[n];
    }
  }
}

// out[t, h*dv + j] = o[t, h, j] / sqrt(mean_j(o[t, h, :]^2) + eps) * gain[h*dv + j] * sigmoid(gate[t, h*dv + j]); a warp per (t, h).
template <typename TO>
__global__ void delta_out_kernel(const float* __restrict__ o, const float* __restrict__ gain, const float* __restrict__ proj,
                                 int ld, int off_g, float eps, TO* __restrict__ out, int rows, int H, int dv) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);     // (t, h)
  if (row >= rows) return;
  const int t = row / H, h = row % H;
  const float* x = o + (size_t)row * dv;
  float ss = 0.f;
  for (int j = lane; j < dv; j += 32) ss = fmaf(x[j], x[j], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  const float* g = proj + (size_t)t * ld + off_g + h * dv;
  for (int j = lane; j < dv; j += 32)
    out[(size_t)row * dv + j] = from_f32<TO>(x[j] * inv * gain[h * dv + j] * sigmoidf_(g[j]));
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_delta_rule_supports(int dk, int dv) { return dk >= 1 && dk <= 256 && dv >= 1 && dv <= 65535 * DR_COLS; }

SLLM_EXPORT int sllm_delta_rule(const float* proj, int ld, int off_r, int off_k, int off_v, int off_a, const float* decay,
                                const float* a_bias, float* state, const int* q_start, const int* state_slots, float* out,
                                int S, int H, int dk, int dv, cudaStream_t stream) {
  SLLM_REQUIRE(S >= 0 && H > 0 && H <= 65535, "delta_rule: bad sizes S=%d H=%d", S, H);
  SLLM_REQUIRE(sllm_delta_rule_supports(dk, dv), "delta_rule: a head of %d key and %d value channels is outside 1..256 keys", dk, dv);
  SLLM_REQUIRE(off_r >= 0 && off_k >= 0 && off_v >= 0 && off_a >= 0 && off_r + H * dk <= ld && off_k + H * dk <= ld &&
                   off_v + H * dv <= ld && off_a + H * dk <= ld, "delta_rule: columns outside the product's %d", ld);
  if (S == 0) return SLLM_OK;
  DeltaParams p;
  p.proj = proj; p.decay = decay; p.a_bias = a_bias; p.state = state; p.q_start = q_start; p.state_slots = state_slots;
  p.out = out; p.ld = ld; p.off_r = off_r; p.off_k = off_k; p.off_v = off_v; p.off_a = off_a; p.H = H; p.dk = dk; p.dv = dv;
  const size_t per_token = (size_t)(5 * dk + DR_COLS + 1) * sizeof(float);
  int chunk = (int)((44 * 1024) / per_token);
  chunk = chunk > DR_MAX_CHUNK ? DR_MAX_CHUNK : (chunk < 1 ? 1 : chunk);
  p.chunk = chunk;
  const size_t smem = per_token * chunk;
  const dim3 grid((unsigned)S, (unsigned)H, (unsigned)((dv + DR_COLS - 1) / DR_COLS));
  if (dk <= 16) launch_kernel(delta_rule_kernel<4>, grid, DR_THREADS, smem, stream, p);
  else if (dk <= 32) launch_kernel(delta_rule_kernel<8>, grid, DR_THREADS, smem, stream, p);
  else if (dk <= 64) launch_kernel(delta_rule_kernel<16>, grid, DR_THREADS, smem, stream, p);
  else if (dk <= 128) launch_kernel(delta_rule_kernel<32>, grid, DR_THREADS, smem, stream, p);
  else launch_kernel(delta_rule_kernel<64>, grid, DR_THREADS, smem, stream, p);
  return launch_status("delta_rule");
}

SLLM_EXPORT int sllm_delta_out(const float* o, const float* gain, const float* proj, int ld, int off_g, float eps, void* out,
                               int out_dtype, int T, int H, int dv, cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && H > 0 && dv > 0 && off_g >= 0 && off_g + H * dv <= ld, "delta_out: bad sizes T=%d H=%d dv=%d", T, H, dv);
  if (T == 0) return SLLM_OK;
  const long rows = (long)T * H;
  const int blocks = (int)((rows + 7) / 8);
  if (out_dtype == SLLM_F32)
    launch_kernel(delta_out_kernel<float>, blocks, 256, 0, stream, o, gain, proj, ld, off_g, eps, (float*)out, (int)rows, H, dv);
  else if (out_dtype == SLLM_BF16)
    launch_kernel(delta_out_kernel<__nv_bfloat16>, blocks, 256, 0, stream, o, gain, proj, ld, off_g, eps, (__nv_bfloat16*)out,
                  (int)rows, H, dv);
  else
    SLLM_REQUIRE(false, "delta_out: unknown dtype %d", out_dtype);
  return launch_status("delta_out");
}
