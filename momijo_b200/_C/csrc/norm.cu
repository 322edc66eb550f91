// LayerNorm and RMSNorm forward/backward for bf16 activations (fp32 statistics).
//
// One CTA per row; each thread keeps up to kVPT 16-byte vectors (8 bf16) of the row in
// registers, so a row is read from HBM exactly once per pass. The forward can fuse the
// residual add that precedes the norm (writes the updated residual stream too). The backward
// is persistent over rows: each CTA keeps its partial dgamma/dbeta in registers, writes one
// partial row per CTA into a scratch buffer, and a second kernel folds the partials.
//
// Replaces the reference's LayerNorm1d, which forms mean/variance with matmul-by-ones on the
// CPU (legacy/src/momijo/learn/nn/layernorm.mojo:27-37). RMSNorm has no counterpart in the
// reference; it follows the same layer style.
#include "common.cuh"

namespace mmj {

constexpr int kNormMaxVPT = 2;

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 q = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z),
         d = unpack_bf16x2(q.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z),
         d = unpack_bf16x2(q.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 q;
  q.x = pack_bf16x2(f[0], f[1]);
  q.y = pack_bf16x2(f[2], f[3]);
  q.z = pack_bf16x2(f[4], f[5]);
  q.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = q;
}

// Block-wide sum of two values. `red` holds 2*32 floats.
__device__ __forceinline__ float2 block_sum2(float a, float b, float* red) {
  a = warp_sum(a);
  b = warp_sum(b);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) { red[warp] = a; red[32 + warp] = b; }
  __syncthreads();
  float x = (lane < nw) ? red[lane] : 0.f;
  float y = (lane < nw) ? red[32 + lane] : 0.f;
  x = warp_sum(x);
  y = warp_sum(y);
  return make_float2(x, y);
}

// mode: 0 = LayerNorm (gamma, beta), 1 = RMSNorm (gamma only)
template <int VPT>
__global__ void norm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                const __nv_bfloat16* __restrict__ res,  // optional residual in
                                __nv_bfloat16* __restrict__ res_out,    // optional x + res out
                                const __nv_bfloat16* __restrict__ gamma,
                                const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                                float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows,
                                int C, float eps, int mode) {
  __shared__ float red[64];
  const int nvec = C >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float v[VPT][8];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      if (vi < nvec) {
        load8(x + (size_t)row * C + vi * 8, v[i]);
        if (res != nullptr) {
          float r[8];
          load8(res + (size_t)row * C + vi * 8, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += r[j];
          // the normalised input is the bf16-rounded residual stream
          if (res_out != nullptr) {
            store8(res_out + (size_t)row * C + vi * 8, v[i]);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16(v[i][j]));
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) { s += v[i][j]; ss += v[i][j] * v[i][j]; }
      }
    }
    float2 t = block_sum2(s, ss, red);
    float mean = 0.f, rstd;
    if (mode == 0) {
      mean = t.x / C;
      // second pass over registers for a numerically safe variance
      float d2 = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = threadIdx.x + i * blockDim.x;
        if (vi < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) { float d = v[i][j] - mean; d2 += d * d; }
        }
      }
      float2 t2 = block_sum2(d2, 0.f, red);
      rstd = rsqrtf(t2.x / C + eps);
    } else {
      rstd = rsqrtf(t.y / C + eps);
    }
    if (threadIdx.x == 0) {
      if (mean_out != nullptr) mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      if (vi < nvec) {
        float g[8], o[8];
        load8(gamma + vi * 8, g);
        if (mode == 0 && beta != nullptr) {
          float b[8];
          load8(beta + vi * 8, b);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd * g[j] + b[j];
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd * g[j];
        }
        store8(y + (size_t)row * C + vi * 8, o);
      }
    }
  }
}

// dx = rstd * (dy*g - mean_c(dy*g) - xhat * mean_c(dy*g*xhat))        (LayerNorm)
// dx = rstd * (dy*g - xhat * mean_c(dy*g*xhat))                          (RMSNorm)
// Optional dres_in is added to dx (gradient arriving through the residual branch).
// kPrefetch: request the next row's vectors before reducing the current one (narrow rows, where a
// CTA is a few warps and several CTAs share an SM; for wide rows the extra registers would cost a
// resident CTA).
template <int VPT, bool kPrefetch>
__global__ void norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                const __nv_bfloat16* __restrict__ x,
                                const __nv_bfloat16* __restrict__ gamma,
                                const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                                const __nv_bfloat16* __restrict__ dres_in,
                                __nv_bfloat16* __restrict__ dx, float* __restrict__ partial_dg,
                                float* __restrict__ partial_db, int rows, int C, int mode) {
  __shared__ float red[64];
  const int nvec = C >> 3;
  float dg[VPT][8], db[VPT][8], g[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = threadIdx.x + i * blockDim.x;
#pragma unroll
    for (int j = 0; j < 8; ++j) { dg[i][j] = 0.f; db[i][j] = 0.f; g[i][j] = 0.f; }
    if (vi < nvec) load8(gamma + vi * 8, g[i]);
  }
  // The next row's vectors are requested before the current row is reduced: with a few rows per
  // CTA in sequence, one row's loads in flight per warp left most of the memory latency exposed.
  uint4 cx[VPT], cdy[VPT], cr[VPT];
  float cmean = 0.f, crstd = 0.f;
  auto fetch = [&](int row, uint4 (&qx)[VPT], uint4 (&qdy)[VPT], uint4 (&qr)[VPT], float& mean,
                   float& rstd) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      qx[i] = qdy[i] = qr[i] = make_uint4(0u, 0u, 0u, 0u);
      if (vi < nvec) {
        qx[i] = *reinterpret_cast<const uint4*>(x + (size_t)row * C + vi * 8);
        qdy[i] = *reinterpret_cast<const uint4*>(dy + (size_t)row * C + vi * 8);
        if (dres_in != nullptr) qr[i] = *reinterpret_cast<const uint4*>(dres_in + (size_t)row * C + vi * 8);
      }
    }
    mean = (mode == 0) ? mean_in[row] : 0.f;
    rstd = rstd_in[row];
  };
  if (kPrefetch && (int)blockIdx.x < rows) fetch(blockIdx.x, cx, cdy, cr, cmean, crstd);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const int nrow = row + gridDim.x;
    uint4 nx[VPT], ndy[VPT], nr[VPT];
    float nmean = 0.f, nrstd = 0.f;
    if (!kPrefetch) {
      fetch(row, cx, cdy, cr, cmean, crstd);
    } else if (nrow < rows) {
      fetch(nrow, nx, ndy, nr, nmean, nrstd);
    } else {
#pragma unroll
      for (int i = 0; i < VPT; ++i) nx[i] = ndy[i] = nr[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    const float mean = cmean, rstd = crstd;
    float xh[VPT][8], gy[VPT][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      if (vi < nvec) {
        float xv[8], dyv[8];
        unpack8(cx[i], xv);
        unpack8(cdy[i], dyv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xv[j] - mean) * rstd;
          gy[i][j] = dyv[j] * g[i][j];
          s1 += gy[i][j];
          s2 += gy[i][j] * xh[i][j];
          dg[i][j] += dyv[j] * xh[i][j];
          db[i][j] += dyv[j];
        }
      }
    }
    float2 t = block_sum2(s1, s2, red);
    const float m1 = (mode == 0) ? t.x / C : 0.f;
    const float m2 = t.y / C;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (gy[i][j] - m1 - xh[i][j] * m2);
        if (dres_in != nullptr) {
          float r[8];
          unpack8(cr[i], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        store8(dx + (size_t)row * C + vi * 8, o);
      }
    }
    if (kPrefetch) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) { cx[i] = nx[i]; cdy[i] = ndy[i]; cr[i] = nr[i]; }
      cmean = nmean;
      crstd = nrstd;
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = threadIdx.x + i * blockDim.x;
    if (vi < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        partial_dg[(size_t)blockIdx.x * C + vi * 8 + j] = dg[i][j];
        if (partial_db != nullptr) partial_db[(size_t)blockIdx.x * C + vi * 8 + j] = db[i][j];
      }
    }
  }
}

// Fold `nparts` partial rows into bf16 gradients (optionally accumulating into existing ones).
__global__ void norm_bwd_finalize_kernel(const float* __restrict__ partial_dg,
                                         const float* __restrict__ partial_db,
                                         __nv_bfloat16* __restrict__ dgamma,
                                         __nv_bfloat16* __restrict__ dbeta, int nparts, int C,
                                         int accumulate) {
  // block (16, 64): 16 adjacent columns (one 64-byte piece per partial row), the partial rows split over
  // threadIdx.y; narrow column strips give 48 CTAs for C = 768 where 32-column strips gave 24 and left
  // the 7 MB of partials to two dozen SMs
  __shared__ float sa[64][17], sb[64][17];
  const int c = blockIdx.x * 16 + threadIdx.x;
  float a = 0.f, b = 0.f;
  if (c < C) {
    for (int p = threadIdx.y; p < nparts; p += 64) {
      a += partial_dg[(size_t)p * C + c];
      if (partial_db != nullptr) b += partial_db[(size_t)p * C + c];
    }
  }
  sa[threadIdx.y][threadIdx.x] = a;
  sb[threadIdx.y][threadIdx.x] = b;
  __syncthreads();
  if (threadIdx.y != 0 || c >= C) return;
  a = 0.f;
  b = 0.f;
#pragma unroll
  for (int y = 0; y < 64; ++y) {
    a += sa[y][threadIdx.x];
    b += sb[y][threadIdx.x];
  }
  if (accumulate) {
    a += __bfloat162float(dgamma[c]);
    if (dbeta != nullptr) b += __bfloat162float(dbeta[c]);
  }
  dgamma[c] = __float2bfloat16(a);
  if (dbeta != nullptr && partial_db != nullptr) dbeta[c] = __float2bfloat16(b);
}

static inline int norm_threads(int C, int vpt) {
  int nvec = C / 8;
  int t = (nvec + vpt - 1) / vpt;
  t = ((t + 31) / 32) * 32;
  return t < 32 ? 32 : t;
}

}  // namespace mmj

using namespace mmj;

// rows x C, C % 8 == 0, C <= 16384. mode 0 LayerNorm, 1 RMSNorm.
MMJ_API int mmj_norm_fwd(const void* x, const void* res, void* res_out, const void* gamma,
                         const void* beta, void* y, float* mean, float* rstd, int rows, int C,
                         float eps, int mode, void* stream) {
  if (C % 8 != 0 || C > 8 * 1024 * kNormMaxVPT) return -1;
  if (rows <= 0) return 0;
  const int vpt = (C / 8 > 1024) ? 2 : 1;
  const int threads = norm_threads(C, vpt);
  const int grid = rows;
  auto xs = (const __nv_bfloat16*)x;
  if (vpt == 1)
    norm_fwd_kernel<1><<<grid, threads, 0, (cudaStream_t)stream>>>(
        xs, (const __nv_bfloat16*)res, (__nv_bfloat16*)res_out, (const __nv_bfloat16*)gamma,
        (const __nv_bfloat16*)beta, (__nv_bfloat16*)y, mean, rstd, rows, C, eps, mode);
  else
    norm_fwd_kernel<2><<<grid, threads, 0, (cudaStream_t)stream>>>(
        xs, (const __nv_bfloat16*)res, (__nv_bfloat16*)res_out, (const __nv_bfloat16*)gamma,
        (const __nv_bfloat16*)beta, (__nv_bfloat16*)y, mean, rstd, rows, C, eps, mode);
  return (int)cudaGetLastError();
}

// Number of partial rows the backward writes (scratch must hold nparts * C floats, twice for
// LayerNorm).
MMJ_API int mmj_norm_bwd_parts(int rows) {
  int n = 148 * 8;
  return rows < n ? rows : n;
}

MMJ_API int mmj_norm_bwd(const void* dy, const void* x, const void* gamma, const float* mean,
                         const float* rstd, const void* dres_in, void* dx, void* dgamma,
                         void* dbeta, float* scratch, int rows, int C, int mode, int accumulate,
                         void* stream) {
  if (C % 8 != 0 || C > 8 * 1024 * kNormMaxVPT) return -1;
  if (rows <= 0) return 0;
  const int vpt = (C / 8 > 1024) ? 2 : 1;
  const int threads = norm_threads(C, vpt);
  const bool prefetch = threads <= 256;
  int nparts = mmj_norm_bwd_parts(rows);  // what the caller sized the scratch for
  if (!prefetch && nparts > 148 * 4) nparts = 148 * 4;
  float* pdg = scratch;
  float* pdb = (mode == 0 && dbeta != nullptr) ? scratch + (size_t)nparts * C : nullptr;
  if (vpt == 1 && prefetch)
    norm_bwd_kernel<1, true><<<nparts, threads, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, mean, rstd,
        (const __nv_bfloat16*)dres_in, (__nv_bfloat16*)dx, pdg, pdb, rows, C, mode);
  else if (vpt == 1)
    norm_bwd_kernel<1, false><<<nparts, threads, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, mean, rstd,
        (const __nv_bfloat16*)dres_in, (__nv_bfloat16*)dx, pdg, pdb, rows, C, mode);
  else
    norm_bwd_kernel<2, false><<<nparts, threads, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, mean, rstd,
        (const __nv_bfloat16*)dres_in, (__nv_bfloat16*)dx, pdg, pdb, rows, C, mode);
  norm_bwd_finalize_kernel<<<(C + 15) / 16, dim3(16, 64), 0, (cudaStream_t)stream>>>(
      pdg, pdb, (__nv_bfloat16*)dgamma, (__nv_bfloat16*)dbeta, nparts, C, accumulate);
  return (int)cudaGetLastError();
}
