// MoE router on the device: softmax over the expert logits, top-k selection, renormalised weights,
// per-expert assignment counts and probability sums, and the load-balance auxiliary loss
//   aux = coef * E * sum_e (count_e / (n * k)) * (psum_e / n)
// in two launches (token pass + a one-block fold), plus the matching backward pass. The reference has no
// mixture-of-experts layer (its layer set is legacy/src/momijo/learn/nn/layers.mojo and nn/*.mojo; its only
// softmax is the last-dimension one, legacy/src/momijo/tensor/math.mojo:447-461); this follows the usual
// top-k softmax router with the Switch-style auxiliary loss.
//
// One warp per token, lane l owns experts l, l + 32, ... (E <= 256). Counts and probability sums are kept
// per warp in shared memory (a lane only ever touches its own experts), folded per block in warp order and
// over the blocks in block order, so the loss and every output are bitwise reproducible.
#include "common.cuh"

namespace mmj {

constexpr int kRouterMaxE = 256;
constexpr int kRouterWarps = 8;
constexpr int kEPL = kRouterMaxE / 32;  // experts per lane

struct TopSel {
  float v;
  int e;
};
__device__ __forceinline__ TopSel warp_argmax(float v, int e) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oe = __shfl_xor_sync(0xffffffffu, e, o);
    if (ov > v || (ov == v && oe < e)) {   // ties go to the lower expert index
      v = ov;
      e = oe;
    }
  }
  return {v, e};
}

// logits [n, ld] bf16; weights [n, k] fp32; idx [n, k] int32; part_cnt / part_psum [grid, E].
__global__ void __launch_bounds__(kRouterWarps * 32)
moe_router_fwd_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int n, int E, int k,
                      float* __restrict__ weights, int* __restrict__ idx, int* __restrict__ part_cnt,
                      float* __restrict__ part_psum) {
  __shared__ float s_psum[kRouterWarps][kRouterMaxE];
  __shared__ int s_cnt[kRouterWarps][kRouterMaxE];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = lane; e < E; e += 32) {
    s_psum[warp][e] = 0.f;
    s_cnt[warp][e] = 0;
  }
  __syncwarp();
  for (long long t = (long long)blockIdx.x * kRouterWarps + warp; t < n; t += (long long)gridDim.x * kRouterWarps) {
    float p[kEPL];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < kEPL; ++j) {
      const int e = lane + 32 * j;
      p[j] = (e < E) ? __bfloat162float(logits[t * ld + e]) : -INFINITY;
      mx = fmaxf(mx, p[j]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kEPL; ++j) {
      p[j] = (lane + 32 * j < E) ? expf(p[j] - mx) : 0.f;
      sum += p[j];
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int j = 0; j < kEPL; ++j) {
      p[j] *= inv;
      if (lane + 32 * j < E) s_psum[warp][lane + 32 * j] += p[j];
    }
    // k rounds of warp arg-max over the values not taken yet
    float q[kEPL];
#pragma unroll
    for (int j = 0; j < kEPL; ++j) q[j] = (lane + 32 * j < E) ? p[j] : -1.f;
    float wsum = 0.f;
    float my_w = 0.f;   // lane i (< k) keeps the i-th selected probability
    int my_e = 0;
    for (int r = 0; r < k; ++r) {
      float bv = -1.f;
      int be = kRouterMaxE;
#pragma unroll
      for (int j = 0; j < kEPL; ++j)
        if (q[j] > bv) {
          bv = q[j];
          be = lane + 32 * j;
        }
      const TopSel s = warp_argmax(bv, be);
      if ((s.e & 31) == lane) {
#pragma unroll
        for (int j = 0; j < kEPL; ++j)
          if (s.e == lane + 32 * j) q[j] = -1.f;
        s_cnt[warp][s.e] += 1;
      }
      if (lane == r) {
        my_w = s.v;
        my_e = s.e;
      }
      wsum += s.v;
    }
    if (lane < k) {
      weights[t * k + lane] = my_w / wsum;
      idx[t * k + lane] = my_e;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float ps = 0.f;
    int c = 0;
    for (int w = 0; w < kRouterWarps; ++w) {
      ps += s_psum[w][e];
      c += s_cnt[w][e];
    }
    part_psum[(long long)blockIdx.x * E + e] = ps;
    part_cnt[(long long)blockIdx.x * E + e] = c;
  }
}

// One block: fold the per-block partials in block order, then the auxiliary loss in expert order.
__global__ void __launch_bounds__(kRouterMaxE)
moe_router_fold_kernel(const int* __restrict__ part_cnt, const float* __restrict__ part_psum, int parts, int E,
                       int n, int k, float coef, int* __restrict__ cnt, float* __restrict__ psum,
                       float* __restrict__ aux) {
  __shared__ float term[kRouterMaxE];
  const int e = threadIdx.x;
  if (e < E) {
    float ps = 0.f;
    int c = 0;
    for (int b = 0; b < parts; ++b) {
      ps += part_psum[(long long)b * E + e];
      c += part_cnt[(long long)b * E + e];
    }
    psum[e] = ps;
    cnt[e] = c;
    term[e] = ((float)c / ((float)n * (float)k)) * (ps / (float)n);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < E; ++i) s += term[i];
    aux[0] = coef * (float)E * s;
  }
}

// dlogits[t, e] = p_e * (dp_e - sum_j p_j dp_j) with
//   dp_e = [e selected] * (dw_e - sum_i dw_i w_i) / s  +  daux * coef * E * f_e / n,
// s = sum of the selected probabilities, f_e = count_e / (n * k) (treated as a constant).
__global__ void __launch_bounds__(kRouterWarps * 32)
moe_router_bwd_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int n, int E, int k,
                      const float* __restrict__ weights, const int* __restrict__ idx,
                      const float* __restrict__ dweights, const float* __restrict__ daux,
                      const int* __restrict__ cnt, float coef, __nv_bfloat16* __restrict__ dlogits,
                      long long ldd) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float da = (daux != nullptr) ? daux[0] : 0.f;
  const float aux_scale = da * coef * (float)E / ((float)n * (float)n * (float)k);
  for (long long t = (long long)blockIdx.x * kRouterWarps + warp; t < n; t += (long long)gridDim.x * kRouterWarps) {
    float p[kEPL];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < kEPL; ++j) {
      const int e = lane + 32 * j;
      p[j] = (e < E) ? __bfloat162float(logits[t * ld + e]) : -INFINITY;
      mx = fmaxf(mx, p[j]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kEPL; ++j) {
      p[j] = (lane + 32 * j < E) ? expf(p[j] - mx) : 0.f;
      sum += p[j];
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    // selected experts: lane i < k holds (e_i, w_i, dw_i)
    const int se = (lane < k) ? idx[t * k + lane] : -1;
    const float sw = (lane < k) ? weights[t * k + lane] : 0.f;
    const float sdw = (dweights != nullptr && lane < k) ? dweights[t * k + lane] : 0.f;
    const float dot = warp_sum(sdw * sw);
    float dp[kEPL];
    float s_sel = 0.f;
#pragma unroll
    for (int j = 0; j < kEPL; ++j) {
      p[j] *= inv;
      const int e = lane + 32 * j;
      dp[j] = (e < E) ? aux_scale * (float)cnt[e] : 0.f;
    }
    // hand each selected (expert, dw) to the lane that owns the expert
    float sel_dw[kEPL];
    bool sel[kEPL];
#pragma unroll
    for (int j = 0; j < kEPL; ++j) { sel_dw[j] = 0.f; sel[j] = false; }
    for (int r = 0; r < k; ++r) {
      const int e = __shfl_sync(0xffffffffu, se, r);
      const float d = __shfl_sync(0xffffffffu, sdw, r);
#pragma unroll
      for (int j = 0; j < kEPL; ++j)
        if (e == lane + 32 * j) {
          sel[j] = true;
          sel_dw[j] = d;
          s_sel += p[j];
        }
    }
    s_sel = warp_sum(s_sel);
    const float inv_s = (s_sel > 0.f) ? 1.0f / s_sel : 0.f;
    float pd = 0.f;
#pragma unroll
    for (int j = 0; j < kEPL; ++j) {
      if (sel[j]) dp[j] += (sel_dw[j] - dot) * inv_s;
      pd += p[j] * dp[j];
    }
    pd = warp_sum(pd);
#pragma unroll
    for (int j = 0; j < kEPL; ++j) {
      const int e = lane + 32 * j;
      if (e < E) dlogits[t * ldd + e] = __float2bfloat16(p[j] * (dp[j] - pd));
    }
  }
}

}  // namespace mmj

using namespace mmj;

MMJ_API int mmj_moe_router_parts() { return 148 * 2; }

// part_cnt / part_psum: scratch of mmj_moe_router_parts() * E entries each.
MMJ_API int mmj_moe_router_fwd(const void* logits, long long ld, int n, int E, int k, float coef, float* weights,
                               int* idx, int* cnt, float* psum, float* aux, int* part_cnt, float* part_psum,
                               void* stream) {
  if (E < 1 || E > kRouterMaxE || k < 1 || k > 32 || k > E || n < 1) return -1;
  int parts = mmj_moe_router_parts();
  const int want = (n + kRouterWarps - 1) / kRouterWarps;
  if (want < parts) parts = want;
  moe_router_fwd_kernel<<<parts, kRouterWarps * 32, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)logits, ld, n, E, k, weights, idx, part_cnt, part_psum);
  moe_router_fold_kernel<<<1, kRouterMaxE, 0, (cudaStream_t)stream>>>(part_cnt, part_psum, parts, E, n, k, coef, cnt,
                                                                      psum, aux);
  return (int)cudaGetLastError();
}

MMJ_API int mmj_moe_router_bwd(const void* logits, long long ld, int n, int E, int k, const float* weights,
                               const int* idx, const float* dweights, const float* daux, const int* cnt,
                               float coef, void* dlogits, long long ldd, void* stream) {
  if (E < 1 || E > kRouterMaxE || k < 1 || k > 32 || n < 1) return -1;
  int grid = 148 * 2;
  const int want = (n + kRouterWarps - 1) / kRouterWarps;
  if (want < grid) grid = want;
  moe_router_bwd_kernel<<<grid, kRouterWarps * 32, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)logits, ld, n, E, k, weights, idx, dweights, daux, cnt, coef,
      (__nv_bfloat16*)dlogits, ldd);
  return (int)cudaGetLastError();
}
