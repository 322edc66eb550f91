// Fused softmax cross-entropy (loss and dlogits in one pass over HBM), the fused AdamW update
// for flat shards (bf16 parameters, fp32 master/m/v), and the gradient norm / non-finite check.
//
// softmax_cross_entropy in the reference returns (loss, dlogits = (softmax - onehot)/N) from a
// single call (legacy/src/momijo/learn/losses/losses.mojo:72-85); this kernel keeps that
// contract and writes dlogits in place over the logits. The AdamW update follows the per-layer
// optimizer rule (legacy/src/momijo/learn/optim/adamw.mojo:105-147, decoupled decay using the
// pre-update weight) rather than the decay-first ordering of the reference's unused GPU kernel
// (legacy/src/momijo/tensor/gpu/runtime.mojo:1134-1172), with an exact sqrtf.
#include "common.cuh"

#include <cstdlib>

namespace mmj {

__device__ __forceinline__ float block_reduce_max(float v, float* red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float x = (lane < nw) ? red[lane] : -INFINITY;
  return warp_max(x);
}
__device__ __forceinline__ float block_reduce_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float x = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(x);
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void unpack_bf16x8(const uint4& q, float (&f)[8]) {
  float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

// One CTA per row. logits: [rows, ld] bf16, columns >= V are padding. When the row fits in
// shared memory (kCache) it is read from HBM once; dlogits overwrite the logits.
//   loss_row[r] = logsumexp(row) - row[target]           (0 for ignored targets)
//   dlogits    = (softmax - onehot) * dscale             (0 in padding and ignored rows)
// Vocab-parallel use: pass vocab_start (first class id held by this shard) and write
// row_max/row_sum partials instead (mode 1), see ce_vp_* below.
template <bool kCache>
__global__ void ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, long long ld, int V,
                                  const long long* __restrict__ targets, float* __restrict__ loss_row,
                                  float dscale, const float* __restrict__ dscale_dev,
                                  long long ignore_index, int write_grad) {
  extern __shared__ __align__(16) uint8_t ce_smem[];
  __shared__ float red[32];
  __nv_bfloat16* cache = reinterpret_cast<__nv_bfloat16*>(ce_smem);
  const long long row = blockIdx.x;
  __nv_bfloat16* g = logits + row * ld;
  const int nvec = (int)(ld >> 3);  // ld % 8 == 0
  const long long tgt = targets[row];
  const bool ignored = (tgt == ignore_index) || !index_ok(tgt, V, /*site=*/3);

  // One pass over the row: running maximum and running sum of exp(x - maximum), rescaled whenever a
  // vector raises the maximum. The exponentials run while later loads are still in flight, instead of
  // in a second pass over the cached row. Everything is in base 2 (one fused multiply-add and one
  // `ex2` per element), and only the vectors that reach past V test their columns.
  constexpr float kL2e = 1.4426950408889634f;
  float mx = -INFINITY, sum = 0.f;
#pragma unroll 4
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 q = reinterpret_cast<const uint4*>(g)[v];
    if (kCache) reinterpret_cast<uint4*>(cache)[v] = q;
    float x[8];
    unpack_bf16x8(q, x);
    if (v * 8 + 8 > V) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (v * 8 + j >= V) x[j] = -INFINITY;
    }
    float vm = fmaxf(fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3])), fmaxf(fmaxf(x[4], x[5]), fmaxf(x[6], x[7])));
    if (vm > mx) {
      sum *= ex2_approx((mx - vm) * kL2e);  // 2^(-inf) = 0 on the first vector
      mx = vm;
    }
    if (mx > -INFINITY) {
      const float nm = -mx * kL2e;
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        s0 += ex2_approx(fmaf(x[j], kL2e, nm));
        s1 += ex2_approx(fmaf(x[j + 1], kL2e, nm));
      }
      sum += s0 + s1;
    }
  }
  const float bmx = block_reduce_max(mx, red);
  sum = (mx > -INFINITY) ? sum * ex2_approx((mx - bmx) * kL2e) : 0.f;
  mx = bmx;
  const __nv_bfloat16* srcp = kCache ? cache : g;
  sum = block_reduce_sum(sum, red);
  const float lse = mx + __logf(sum);
  if (threadIdx.x == 0) {
    float l = 0.f;
    if (!ignored) l = lse - __bfloat162float(srcp[tgt]);
    loss_row[row] = l;
  }
  if (!write_grad) return;
  __syncthreads();  // everyone has read srcp[tgt] before the in-place overwrite (non-cached path)
  const float sc = ignored ? 0.f : dscale * (dscale_dev != nullptr ? *dscale_dev : 1.0f);
  if (sc == 0.f) {
    for (int v = threadIdx.x; v < nvec; v += blockDim.x)
      reinterpret_cast<uint4*>(g)[v] = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  // dlogit = softmax * sc = sign(sc) * 2^(x * log2(e) - lse * log2(e) + log2|sc|): the normaliser and the
  // scale ride in the exponent's offset
  const float off = -lse * kL2e + __log2f(fabsf(sc));
  const float sgn = sc < 0.f ? -1.f : 1.f;
  const int tv = (int)(tgt >> 3), tj = (int)(tgt & 7);
#pragma unroll 2
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 q = reinterpret_cast<const uint4*>(srcp)[v];
    float x[8], o[8];
    unpack_bf16x8(q, x);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = ex2_approx(fmaf(x[j], kL2e, off));
    if (sgn < 0.f) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = -o[j];
    }
    if (v * 8 + 8 > V) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (v * 8 + j >= V) o[j] = 0.f;
    }
    if (v == tv) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j == tj) o[j] -= sc;
    }
    uint4 w;
    w.x = pack_bf16x2(o[0], o[1]);
    w.y = pack_bf16x2(o[2], o[3]);
    w.z = pack_bf16x2(o[4], o[5]);
    w.w = pack_bf16x2(o[6], o[7]);
    reinterpret_cast<uint4*>(g)[v] = w;
  }
}

// Vocab-parallel cross-entropy, phase 1: per-shard row max, sum(exp(x - max)) and the target
// logit (if the target lives in this shard). Ranks then combine (max, sum, tgt) across the
// tensor-parallel group with a tiny all-reduce and call phase 2.
__global__ void ce_vp_stats_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int Vloc,
                                   long long vocab_start, const long long* __restrict__ targets,
                                   float* __restrict__ row_max, float* __restrict__ row_sum,
                                   float* __restrict__ row_tgt) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* g = logits + row * ld;
  const int nvec = (int)(ld >> 3);
  float mx = -INFINITY;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 q = reinterpret_cast<const uint4*>(g)[v];
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&q);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (v * 8 + j < Vloc) mx = fmaxf(mx, __bfloat162float(e[j]));
  }
  mx = block_reduce_max(mx, red);
  float sum = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 q = reinterpret_cast<const uint4*>(g)[v];
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&q);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (v * 8 + j < Vloc) sum += __expf(__bfloat162float(e[j]) - mx);
  }
  sum = block_reduce_sum(sum, red);
  if (threadIdx.x == 0) {
    row_max[row] = mx;
    row_sum[row] = sum;
    const long long t = targets[row] - vocab_start;
    row_tgt[row] = (t >= 0 && t < Vloc) ? __bfloat162float(g[t]) : 0.f;
  }
}
// Phase 2: dlogits = (exp(x - gmax)/gsum - onehot) * dscale, in place.
__global__ void ce_vp_grad_kernel(__nv_bfloat16* __restrict__ logits, long long ld, int Vloc,
                                  long long vocab_start, const long long* __restrict__ targets,
                                  const float* __restrict__ gmax, const float* __restrict__ gsum,
                                  float dscale, const float* __restrict__ dscale_dev) {
  if (dscale_dev != nullptr) dscale *= *dscale_dev;   // gradient of the loss, folded in here (no extra pass)
  const long long row = blockIdx.x;
  __nv_bfloat16* g = logits + row * ld;
  const int nvec = (int)(ld >> 3);
  const float mx = gmax[row];
  const float inv = 1.0f / gsum[row];
  const long long t = targets[row] - vocab_start;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 q = reinterpret_cast<const uint4*>(g)[v];
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&q);
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = v * 8 + j;
      float p = (c < Vloc) ? __expf(__bfloat162float(e[j]) - mx) * inv : 0.f;
      if (c == t) p -= 1.f;
      o[j] = p * dscale;
    }
    uint4 w;
    w.x = pack_bf16x2(o[0], o[1]);
    w.y = pack_bf16x2(o[2], o[3]);
    w.z = pack_bf16x2(o[4], o[5]);
    w.w = pack_bf16x2(o[6], o[7]);
    reinterpret_cast<uint4*>(g)[v] = w;
  }
}

// Deterministic mean (or sum) of n floats into out[0]; single CTA.
__global__ void reduce_mean_kernel(const float* __restrict__ x, float* __restrict__ out,
                                   long long n, float scale, const float* __restrict__ scale_dev) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) s += x[i];
  s = block_reduce_sum(s, red);
  if (threadIdx.x == 0) out[0] = s * scale * (scale_dev != nullptr ? *scale_dev : 1.0f);
}

// out[0] = 1 / max(1, number of targets that differ from ignore_index): the factor of a mean over
// the rows that count. Single CTA; runs before the cross-entropy kernel, which reads the factor.
__global__ void ce_count_valid_kernel(const long long* __restrict__ targets, long long n,
                                      long long ignore_index, float* __restrict__ out) {
  __shared__ float red[32];
  float c = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) c += (targets[i] != ignore_index) ? 1.f : 0.f;
  c = block_reduce_sum(c, red);
  if (threadIdx.x == 0) out[0] = 1.0f / fmaxf(c, 1.0f);
}

// ---- fused AdamW over a flat shard -------------------------------------------------------------
// g: gradient (bf16 or fp32), w: fp32 master, m/v: fp32 moments, p_out: bf16 parameter copy.
//   g' = g * grad_scale;  m = b1 m + (1-b1) g';  v = b2 v + (1-b2) g'^2
//   w  = w - lr * ( (m/bc1) / (sqrt(v/bc2) + eps) + wd * w )
// The whole update is skipped when *found_inf != 0 (GradScaler protocol).
template <typename GT>
__global__ void adamw_kernel(const GT* __restrict__ g, float* __restrict__ w, float* __restrict__ m,
                             float* __restrict__ v, __nv_bfloat16* __restrict__ p_out, long long n,
                             float lr, float b1, float b2, float eps, float wd, float bc1,
                             float bc2, float grad_scale, const float* __restrict__ grad_scale_dev,
                             const int* __restrict__ found_inf) {
  if (found_inf != nullptr && *found_inf != 0) return;
  if (grad_scale_dev != nullptr) grad_scale *= *grad_scale_dev;
  const float inv_bc1 = 1.0f / bc1, inv_bc2 = 1.0f / bc2;
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < n;
       i += (long long)gridDim.x * blockDim.x * 4) {
    if (i + 4 <= n) {
      float gg[4];
      if (sizeof(GT) == 2) {
        uint2 q = *reinterpret_cast<const uint2*>(g + i);
        float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y);
        gg[0] = a.x; gg[1] = a.y; gg[2] = b.x; gg[3] = b.y;
      } else {
        float4 q = *reinterpret_cast<const float4*>(g + i);
        gg[0] = q.x; gg[1] = q.y; gg[2] = q.z; gg[3] = q.w;
      }
      float4 wv = *reinterpret_cast<float4*>(w + i);
      float4 mv = *reinterpret_cast<float4*>(m + i);
      float4 vv = *reinterpret_cast<float4*>(v + i);
      float ww[4] = {wv.x, wv.y, wv.z, wv.w}, mm[4] = {mv.x, mv.y, mv.z, mv.w},
            v2[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gj = gg[j] * grad_scale;
        mm[j] = b1 * mm[j] + (1.f - b1) * gj;
        v2[j] = b2 * v2[j] + (1.f - b2) * gj * gj;
        const float upd = (mm[j] * inv_bc1) / (sqrtf(v2[j] * inv_bc2) + eps);
        ww[j] = ww[j] - lr * (upd + wd * ww[j]);
      }
      *reinterpret_cast<float4*>(w + i) = make_float4(ww[0], ww[1], ww[2], ww[3]);
      *reinterpret_cast<float4*>(m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(v + i) = make_float4(v2[0], v2[1], v2[2], v2[3]);
      if (p_out != nullptr) {
        uint2 o;
        o.x = pack_bf16x2(ww[0], ww[1]);
        o.y = pack_bf16x2(ww[2], ww[3]);
        *reinterpret_cast<uint2*>(p_out + i) = o;
      }
    } else {
      for (long long k = i; k < n; ++k) {
        float gj = (sizeof(GT) == 2) ? __bfloat162float(((const __nv_bfloat16*)g)[k])
                                     : ((const float*)g)[k];
        gj *= grad_scale;
        float mk = b1 * m[k] + (1.f - b1) * gj;
        float vk = b2 * v[k] + (1.f - b2) * gj * gj;
        float wk = w[k];
        wk = wk - lr * ((mk * inv_bc1) / (sqrtf(vk * inv_bc2) + eps) + wd * wk);
        m[k] = mk; v[k] = vk; w[k] = wk;
        if (p_out != nullptr) p_out[k] = __float2bfloat16(wk);
      }
    }
  }
}

// SGD with optional momentum and weight decay on a flat fp32 buffer (bf16 or fp32 grads).
template <typename GT>
__global__ void sgd_kernel(const GT* __restrict__ g, float* __restrict__ w, float* __restrict__ mom,
                           __nv_bfloat16* __restrict__ p_out, long long n, float lr, float momentum,
                           float wd, float grad_scale) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float gj = (sizeof(GT) == 2) ? __bfloat162float(((const __nv_bfloat16*)g)[i]) : ((const float*)g)[i];
    gj = gj * grad_scale + wd * w[i];
    if (mom != nullptr) {
      const float b = momentum * mom[i] + gj;
      mom[i] = b;
      gj = b;
    }
    const float wk = w[i] - lr * gj;
    w[i] = wk;
    if (p_out != nullptr) p_out[i] = __float2bfloat16(wk);
  }
}

// ---- squared norm + non-finite detection --------------------------------------------------------
// Stage 1 writes one partial per CTA into scratch[gridDim.x]; stage 2 folds them into
// out[0] = sum of squares and sets found_inf[0] = 1 if any element is inf/nan.
template <typename T>
__global__ void sqnorm_partial_kernel(const T* __restrict__ x, long long n, float* __restrict__ scratch,
                                      int* __restrict__ found_inf) {
  __shared__ float red[32];
  float s = 0.f;
  bool bad = false;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float f = (sizeof(T) == 2) ? __bfloat162float(((const __nv_bfloat16*)x)[i]) : ((const float*)x)[i];
    s += f * f;
    bad |= !isfinite(f);
  }
  s = block_reduce_sum(s, red);
  if (threadIdx.x == 0) scratch[blockIdx.x] = s;
  if (bad && found_inf != nullptr) atomicExch(found_inf, 1);
}
__global__ void sqnorm_finalize_kernel(const float* __restrict__ scratch, int nparts,
                                       float* __restrict__ out, int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += scratch[i];
  s = block_reduce_sum(s, red);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
}

}  // namespace mmj

using namespace mmj;
#define STREAM ((cudaStream_t)stream)

static bool g_ce_attr = false;

// logits [rows, ld] bf16 (ld % 8 == 0, V <= ld); targets int64; loss_row [rows] fp32.
MMJ_API int mmj_ce_fwd_bwd(void* logits, long long ld, int V, const long long* targets,
                           float* loss_row, long long rows, float dscale, const float* dscale_dev,
                           long long ignore_index, int write_grad, void* stream) {
  if (ld % 8 || V > ld) return -1;
  if (rows == 0) return 0;
  const size_t bytes = (size_t)ld * 2;
  // Default: no shared-memory copy of the row, 512 threads, four CTAs per SM; the write pass re-reads
  // the row, which is still in L2 (a few hundred rows are in flight). Measured at 16384 x 50257:
  // 0.75 ms against 1.04 ms for the variant that caches the row in shared memory (two CTAs per SM,
  // whose load, exp and store phases then overlap poorly). MOMIJO_CE_MODE=0 selects the cached variant.
  static int ce_mode = -1;
  if (ce_mode < 0) {
    const char* e = getenv("MOMIJO_CE_MODE");
    ce_mode = e ? atoi(e) : 1;
  }
  if (ce_mode != 0) {
    ce_fwd_bwd_kernel<false><<<(unsigned)rows, 512, 0, STREAM>>>(
        (__nv_bfloat16*)logits, ld, V, targets, loss_row, dscale, dscale_dev, ignore_index, write_grad);
    return (int)cudaGetLastError();
  }
  if (bytes <= 200 * 1024) {
    if (!g_ce_attr) {
      cudaFuncSetAttribute(ce_fwd_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           200 * 1024);
      g_ce_attr = true;
    }
    ce_fwd_bwd_kernel<true><<<(unsigned)rows, 512, bytes, STREAM>>>(
        (__nv_bfloat16*)logits, ld, V, targets, loss_row, dscale, dscale_dev, ignore_index, write_grad);
  } else {
    ce_fwd_bwd_kernel<false><<<(unsigned)rows, 1024, 0, STREAM>>>(
        (__nv_bfloat16*)logits, ld, V, targets, loss_row, dscale, dscale_dev, ignore_index, write_grad);
  }
  return (int)cudaGetLastError();
}
MMJ_API int mmj_ce_vp_stats(const void* logits, long long ld, int Vloc, long long vocab_start,
                            const long long* targets, float* row_max, float* row_sum,
                            float* row_tgt, long long rows, void* stream) {
  if (ld % 8 || Vloc > ld) return -1;
  if (rows == 0) return 0;
  ce_vp_stats_kernel<<<(unsigned)rows, 512, 0, STREAM>>>((const __nv_bfloat16*)logits, ld, Vloc,
                                                         vocab_start, targets, row_max, row_sum,
                                                         row_tgt);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_ce_vp_grad(void* logits, long long ld, int Vloc, long long vocab_start,
                           const long long* targets, const float* gmax, const float* gsum,
                           long long rows, float dscale, const float* dscale_dev, void* stream) {
  if (ld % 8 || Vloc > ld) return -1;
  if (rows == 0) return 0;
  ce_vp_grad_kernel<<<(unsigned)rows, 512, 0, STREAM>>>((__nv_bfloat16*)logits, ld, Vloc,
                                                        vocab_start, targets, gmax, gsum, dscale, dscale_dev);
  return (int)cudaGetLastError();
}
// out[0] = scale * (*scale_dev, when given) * sum(x)
MMJ_API int mmj_reduce_mean(const float* x, float* out, long long n, float scale,
                            const float* scale_dev, void* stream) {
  reduce_mean_kernel<<<1, 1024, 0, STREAM>>>(x, out, n, scale, scale_dev);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_ce_count_valid(const long long* targets, long long n, long long ignore_index,
                               float* out_inv, void* stream) {
  ce_count_valid_kernel<<<1, 1024, 0, STREAM>>>(targets, n, ignore_index, out_inv);
  return (int)cudaGetLastError();
}

static inline int grid_for4(long long n) {
  long long g = ((n + 3) / 4 + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  return g < 1 ? 1 : (int)g;
}

// grad_dtype: 0 bf16, 1 fp32
MMJ_API int mmj_adamw(const void* g, int grad_dtype, float* w, float* m, float* v, void* p_out,
                      long long n, float lr, float b1, float b2, float eps, float wd, float bc1,
                      float bc2, float grad_scale, const float* grad_scale_dev,
                      const int* found_inf, void* stream) {
  if (n == 0) return 0;
  if (grad_dtype == 0)
    adamw_kernel<__nv_bfloat16><<<grid_for4(n), 256, 0, STREAM>>>(
        (const __nv_bfloat16*)g, w, m, v, (__nv_bfloat16*)p_out, n, lr, b1, b2, eps, wd, bc1, bc2,
        grad_scale, grad_scale_dev, found_inf);
  else
    adamw_kernel<float><<<grid_for4(n), 256, 0, STREAM>>>((const float*)g, w, m, v,
                                                          (__nv_bfloat16*)p_out, n, lr, b1, b2, eps,
                                                          wd, bc1, bc2, grad_scale, grad_scale_dev,
                                                          found_inf);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_sgd(const void* g, int grad_dtype, float* w, float* mom, void* p_out, long long n,
                    float lr, float momentum, float wd, float grad_scale, void* stream) {
  if (n == 0) return 0;
  long long gr = (n + 255) / 256;
  if (gr > 148 * 8) gr = 148 * 8;
  if (grad_dtype == 0)
    sgd_kernel<__nv_bfloat16><<<(int)gr, 256, 0, STREAM>>>((const __nv_bfloat16*)g, w, mom,
                                                           (__nv_bfloat16*)p_out, n, lr, momentum, wd,
                                                           grad_scale);
  else
    sgd_kernel<float><<<(int)gr, 256, 0, STREAM>>>((const float*)g, w, mom, (__nv_bfloat16*)p_out, n,
                                                   lr, momentum, wd, grad_scale);
  return (int)cudaGetLastError();
}

// scratch must hold mmj_sqnorm_parts() floats. dtype: 0 bf16, 1 fp32.
MMJ_API int mmj_sqnorm_parts() { return 148 * 4; }
MMJ_API int mmj_sqnorm(const void* x, int dtype, long long n, float* scratch, float* out,
                       int* found_inf, int accumulate, void* stream) {
  const int parts = mmj_sqnorm_parts();
  if (dtype == 0)
    sqnorm_partial_kernel<__nv_bfloat16><<<parts, 256, 0, STREAM>>>((const __nv_bfloat16*)x, n,
                                                                   scratch, found_inf);
  else
    sqnorm_partial_kernel<float><<<parts, 256, 0, STREAM>>>((const float*)x, n, scratch, found_inf);
  sqnorm_finalize_kernel<<<1, 256, 0, STREAM>>>(scratch, parts, out, accumulate);
  return (int)cudaGetLastError();
}

MMJ_BOUNDS_READER(mmj_debug_bounds_loss)
