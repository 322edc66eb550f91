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
  pdl_wait();
  pdl_trigger();
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

// ---- streamed kernels: rows arrive through a shared-memory ring filled by bulk copies ------------
//
// One persistent CTA of sixteen warps per SM. Tiles of 16 / G consecutive rows (contiguous in
// memory) are fetched by one `cp.async.bulk` per tensor, completion counted on the stage's
// mbarrier; lane 0 of warp 0 issues them, S - 1 tiles ahead of the tile being consumed, so the bytes
// in flight per SM are those of the ring and not of the registers. G warps share a row, each lane
// holding NV 16-byte vectors of it; with G = 1 (rows up to 1024 columns) a row is reduced by
// shuffles alone. Sixteen warps (four per scheduler) are what hides the shuffle and
// shared-memory latencies of a row: with eight the kernels issued on 40 % of the cycles and stayed
// at half of the copy bandwidth. The backward therefore keeps nothing of a row in registers between
// its two passes (it reads the tile from shared memory twice and frees the stage afterwards), which
// leaves room for the dgamma / dbeta sums at 128 registers per thread. Those sums are folded across
// the warps through the (by then idle) ring and leave as ONE partial row per CTA, so the second
// kernel reads at most 148 rows.
constexpr int kNormWarps = 16;
constexpr int kNormMaxStages = 6;
constexpr int kNormThreads = kNormWarps * 32;

__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes,
                                             uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes),
        "r"(smem_u32(bar))
      : "memory");
}

struct NormRing {
  int stages;        // ring depth
  int tile_rows;     // rows per tile = kNormWarps / G
  int tensor_bytes;  // tile_rows * C * 2, rounded up to 128
};

// After a wait gave up: give the copies that were already requested a bounded time to land, so
// that the CTA does not retire with bulk copies in flight into its shared memory.
__device__ __forceinline__ void drain_ring(uint64_t* full, int stages, int issued) {
  for (int k = issued > stages ? issued - stages : 0; k < issued; ++k) {
    const int s = k % stages;
    const uint32_t parity = (k / stages) & 1;
    for (int spin = 0; spin < (1 << 20); ++spin)
      if (mbar_try_wait(&full[s], parity)) break;
  }
}

// Sum of (a, b) over the G warps that share a row. `red` has room for one float2 per warp and two
// alternating halves, so that one CTA barrier per use is enough.
template <int G>
__device__ __forceinline__ float2 group_sum2(float a, float b, float2* red, int warp, int& flip) {
  a = warp_sum(a);
  b = warp_sum(b);
  if (G == 1) return make_float2(a, b);
  float2* r = red + flip * kNormWarps;
  flip ^= 1;
  if ((threadIdx.x & 31) == 0) r[warp] = make_float2(a, b);
  __syncthreads();
  const int g0 = (warp / G) * G;
  float x = 0.f, y = 0.f;
#pragma unroll
  for (int i = 0; i < G; ++i) { x += r[g0 + i].x; y += r[g0 + i].y; }
  return make_float2(x, y);
}

template <int G>
__device__ __forceinline__ float group_sum1(float a, float2* red, int warp, int& flip) {
  a = warp_sum(a);
  if (G == 1) return a;
  float2* r = red + flip * kNormWarps;
  flip ^= 1;
  if ((threadIdx.x & 31) == 0) r[warp].x = a;
  __syncthreads();
  const int g0 = (warp / G) * G;
  float x = 0.f;
#pragma unroll
  for (int i = 0; i < G; ++i) x += r[g0 + i].x;
  return x;
}

// The copies of this CTA's `k`-th tile (global tile k * gridDim.x + blockIdx.x) into its stage.
struct NormFetch {
  const __nv_bfloat16* src[3];
  int ntens, rows, C;
  NormRing ring;
  uint8_t* smem;
  uint64_t* full;
  __device__ __forceinline__ void issue(int k) const {
    const int s = k % ring.stages;
    const int r0 = (k * (int)gridDim.x + (int)blockIdx.x) * ring.tile_rows;
    const int nr = min(ring.tile_rows, rows - r0);
    const uint32_t bytes = (uint32_t)nr * C * 2;
    uint8_t* dst = smem + (size_t)s * ntens * ring.tensor_bytes;
    mbar_expect_tx(&full[s], bytes * ntens);
#pragma unroll
    for (int t = 0; t < 3; ++t)  // constant indices keep `src` in registers
      if (t < ntens)
        bulk_load_1d(dst + (size_t)t * ring.tensor_bytes, src[t] + (size_t)r0 * C, bytes, &full[s]);
  }
};

template <int NV, int G>
__global__ void __launch_bounds__(kNormThreads, 1)
norm_fwd_stream_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                       __nv_bfloat16* __restrict__ res_out, const __nv_bfloat16* __restrict__ gamma,
                       const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                       float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int C,
                       float eps, int mode, NormRing ring, int* status) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint64_t full[kNormMaxStages], empty[kNormMaxStages];
  __shared__ float2 red[2 * kNormWarps];
  __shared__ int abort_flag, issued_sh;
  pdl_wait();  // the set-up below already requests the first tiles
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntiles = (rows + ring.tile_rows - 1) / ring.tile_rows;
  const int my_tiles = (ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  NormFetch fetch{{x, res, nullptr}, res != nullptr ? 2 : 1, rows, C, ring, smem, full};
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < ring.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], kNormWarps); }
    mbar_fence_init();
    int k = 0;
    for (; k < my_tiles && k < ring.stages - 1; ++k) fetch.issue(k);
    issued_sh = k;
  }
  __syncthreads();
  const int grp = warp / G, sub = warp % G;
  const int nvec = C >> 3;
  // gamma / beta of this lane's columns stay in registers (packed) for the whole kernel
  uint4 gq[NV], bq[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = (sub * NV + i) * 32 + lane;
    gq[i] = bq[i] = make_uint4(0u, 0u, 0u, 0u);
    if (vi < nvec) {
      gq[i] = *reinterpret_cast<const uint4*>(gamma + vi * 8);
      if (mode == 0 && beta != nullptr) bq[i] = *reinterpret_cast<const uint4*>(beta + vi * 8);
    }
  }
  const float invC = 1.f / C;
  int flip = 0;
  bool dead = false;
  for (int it = 0; it < my_tiles; ++it) {
    const int s = it % ring.stages;
    if (threadIdx.x == 0 && !dead) {
      // keep S - 1 tiles ahead: tile it + S - 1 goes into the stage that tile it - 1 used
      const int k = it + ring.stages - 1;
      if (k < my_tiles) {
        if (it == 0 || mbar_wait(&empty[k % ring.stages], ((it - 1) / ring.stages) & 1, &abort_flag, status,
                                 kTimeoutEmpty, it)) {
          fetch.issue(k);
          issued_sh = k + 1;
        }
      }
    }
    __syncwarp();
    if (!dead && !mbar_wait_warp(&full[s], (it / ring.stages) & 1, &abort_flag, status, kTimeoutFull, it))
      dead = true;
    if (dead) {
      // a warp whose wait gave up still meets the others at the row-sum barriers
      if (G == 1) break;
      __syncthreads();
      if (mode == 0) __syncthreads();
      continue;
    }
    const int row = (it * (int)gridDim.x + (int)blockIdx.x) * ring.tile_rows + grp;
    const bool live = row < rows;
    const uint8_t* st = smem + (size_t)s * fetch.ntens * ring.tensor_bytes + (size_t)grp * C * 2;
    float v[NV][8];
    float sum = 0.f, sq = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = (sub * NV + i) * 32 + lane;
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
      if (live && vi < nvec) {
        unpack8(*reinterpret_cast<const uint4*>(st + vi * 16), v[i]);
        if (res != nullptr) {
          float r[8];
          unpack8(*reinterpret_cast<const uint4*>(st + ring.tensor_bytes + vi * 16), r);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += r[j];
          if (res_out != nullptr) {
            // the normalised input is the bf16-rounded residual stream
            store8(res_out + (size_t)row * C + vi * 8, v[i]);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16(v[i][j]));
          }
        }
        float s0 = 0.f, q0 = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) { s0 += v[i][j]; q0 = fmaf(v[i][j], v[i][j], q0); }
        sum += s0;
        sq += q0;
      }
    }
    // the tile is in registers: hand the stage back before the arithmetic
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
    float2 t = group_sum2<G>(sum, sq, red, warp, flip);
    float mean = 0.f, rstd;
    if (mode == 0) {
      mean = t.x * invC;
      float d2 = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int vi = (sub * NV + i) * 32 + lane;
        if (live && vi < nvec) {
          float p = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) { const float d = v[i][j] - mean; p = fmaf(d, d, p); }
          d2 += p;
        }
      }
      rstd = rsqrtf(group_sum1<G>(d2, red, warp, flip) * invC + eps);
    } else {
      rstd = rsqrtf(t.y * invC + eps);
    }
    if (live) {
      if (lane == 0 && sub == 0) {
        if (mean_out != nullptr) mean_out[row] = mean;
        rstd_out[row] = rstd;
      }
      const float nmr = -mean * rstd;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int vi = (sub * NV + i) * 32 + lane;
        if (vi < nvec) {
          float g[8], b[8], o[8];
          unpack8(gq[i], g);
          unpack8(bq[i], b);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = fmaf(fmaf(v[i][j], rstd, nmr), g[j], b[j]);
          store8(y + (size_t)row * C + vi * 8, o);
        }
      }
    }
  }
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) drain_ring(full, ring.stages, issued_sh);
}

template <int NV, int G, bool kBeta>
__global__ void __launch_bounds__(kNormThreads, 1)
norm_bwd_stream_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                       const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                       const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres_in,
                       __nv_bfloat16* __restrict__ dx, float* __restrict__ partial_dg,
                       float* __restrict__ partial_db, int rows, int C, int mode, NormRing ring,
                       int* status) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint64_t full[kNormMaxStages], empty[kNormMaxStages];
  __shared__ float2 red[2 * kNormWarps];
  __shared__ int abort_flag, issued_sh;
  pdl_wait();  // the set-up below already requests the first tiles
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntiles = (rows + ring.tile_rows - 1) / ring.tile_rows;
  const int my_tiles = (ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  NormFetch fetch{{x, dy, dres_in}, dres_in != nullptr ? 3 : 2, rows, C, ring, smem, full};
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < ring.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], kNormWarps); }
    mbar_fence_init();
    int k = 0;
    for (; k < my_tiles && k < ring.stages - 1; ++k) fetch.issue(k);
    issued_sh = k;
  }
  __syncthreads();
  const int grp = warp / G, sub = warp % G;
  const int nvec = C >> 3;
  float dg[NV][8], db[kBeta ? NV : 1][8];
  uint4 gq[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dg[i][j] = 0.f;
      if (kBeta) db[i][j] = 0.f;
    }
    const int vi = (sub * NV + i) * 32 + lane;
    gq[i] = make_uint4(0u, 0u, 0u, 0u);
    if (vi < nvec) gq[i] = *reinterpret_cast<const uint4*>(gamma + vi * 8);
  }
  const float invC = 1.f / C;
  int flip = 0;
  bool dead = false;
  for (int it = 0; it < my_tiles; ++it) {
    const int s = it % ring.stages;
    if (threadIdx.x == 0 && !dead) {
      const int k = it + ring.stages - 1;
      if (k < my_tiles) {
        if (it == 0 || mbar_wait(&empty[k % ring.stages], ((it - 1) / ring.stages) & 1, &abort_flag, status,
                                 kTimeoutEmpty, it)) {
          fetch.issue(k);
          issued_sh = k + 1;
        }
      }
    }
    __syncwarp();
    if (!dead && !mbar_wait_warp(&full[s], (it / ring.stages) & 1, &abort_flag, status, kTimeoutFull, it))
      dead = true;
    if (dead) {
      if (G == 1) break;
      __syncthreads();
      continue;
    }
    const int row = (it * (int)gridDim.x + (int)blockIdx.x) * ring.tile_rows + grp;
    const bool live = row < rows;
    const uint8_t* st = smem + (size_t)s * fetch.ntens * ring.tensor_bytes + (size_t)grp * C * 2;
    const float mean = (live && mode == 0) ? mean_in[row] : 0.f;
    const float rstd = live ? rstd_in[row] : 0.f;
    // xh = x * rstd + nmr keeps the subtraction inside one fused multiply-add
    const float nmr = -mean * rstd;
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = (sub * NV + i) * 32 + lane;
      if (live && vi < nvec) {
        float xv[8], dyv[8], g[8];
        unpack8(*reinterpret_cast<const uint4*>(st + vi * 16), xv);
        unpack8(*reinterpret_cast<const uint4*>(st + ring.tensor_bytes + vi * 16), dyv);
        unpack8(gq[i], g);
        float a1 = 0.f, a2 = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = fmaf(xv[j], rstd, nmr);
          const float gy = dyv[j] * g[j];
          a1 += gy;
          a2 = fmaf(gy, xh, a2);
          dg[i][j] = fmaf(dyv[j], xh, dg[i][j]);
          if (kBeta) db[i][j] += dyv[j];
        }
        s1 += a1;
        s2 += a2;
      }
    }
    float2 t = group_sum2<G>(s1, s2, red, warp, flip);
    if (live) {
      // dx = rstd * (gy - m1 - xh * m2), with the two row means folded into the constants; the
      // row is read from the stage a second time instead of being held in registers
      const float c1 = (mode == 0) ? -t.x * invC * rstd : 0.f;
      const float c2 = -t.y * invC * rstd;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int vi = (sub * NV + i) * 32 + lane;
        if (vi < nvec) {
          float xv[8], dyv[8], g[8], o[8];
          unpack8(*reinterpret_cast<const uint4*>(st + vi * 16), xv);
          unpack8(*reinterpret_cast<const uint4*>(st + ring.tensor_bytes + vi * 16), dyv);
          unpack8(gq[i], g);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float xh = fmaf(xv[j], rstd, nmr);
            o[j] = fmaf(dyv[j] * g[j], rstd, fmaf(xh, c2, c1));
          }
          if (dres_in != nullptr) {
            float r[8];
            unpack8(*reinterpret_cast<const uint4*>(st + 2 * ring.tensor_bytes + vi * 16), r);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] += r[j];
          }
          store8(dx + (size_t)row * C + vi * 8, o);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
  }
  // Fold the warps' column sums: every bulk copy this CTA asked for has landed (each tile was
  // waited for by all warps) unless a wait gave up, in which case nothing more is written.
  __syncthreads();
  if (abort_flag) {
    if (threadIdx.x == 0) drain_ring(full, ring.stages, issued_sh);
    return;
  }
  float* fold = reinterpret_cast<float*>(smem);  // [groups][C] dgamma, then [groups][C] dbeta
  constexpr int kGroups = kNormWarps / G;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = (sub * NV + i) * 32 + lane;
    if (vi < nvec) {
#pragma unroll
      for (int j = 0; j < 8; j += 4) {
        *reinterpret_cast<float4*>(fold + (size_t)grp * C + vi * 8 + j) =
            make_float4(dg[i][j], dg[i][j + 1], dg[i][j + 2], dg[i][j + 3]);
        if (kBeta)
          *reinterpret_cast<float4*>(fold + (size_t)(kGroups + grp) * C + vi * 8 + j) =
              make_float4(db[i][j], db[i][j + 1], db[i][j + 2], db[i][j + 3]);
      }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int g = 0; g < kGroups; ++g) {
      a += fold[(size_t)g * C + c];
      if (kBeta) b += fold[(size_t)(kGroups + g) * C + c];
    }
    partial_dg[(size_t)blockIdx.x * C + c] = a;
    if (kBeta) partial_db[(size_t)blockIdx.x * C + c] = b;
  }
}

// Ring geometry for C columns and `ntens` streamed tensors; stages == 0 when the rows do not fit.
static inline NormRing norm_ring(int C, int G, int ntens, bool fold) {
  NormRing r;
  r.tile_rows = kNormWarps / G;
  r.tensor_bytes = ((r.tile_rows * C * 2 + 127) / 128) * 128;
  const int budget = 226 * 1024;
  int stages = budget / (r.tensor_bytes * ntens);
  r.stages = stages > kNormMaxStages ? kNormMaxStages : stages;
  if (r.stages < 3) r.stages = 0;  // one tile being read, two on their way
  // the backward reuses the ring for the fold of the column sums
  if (fold && (size_t)2 * r.tile_rows * C * 4 > (size_t)r.stages * ntens * r.tensor_bytes) r.stages = 0;
  return r;
}

// Warps per row and vectors per lane for C columns: a lane holds at most four vectors, rows up to
// 1024 columns stay inside one warp, 8192 columns take eight warps.
static inline bool norm_split(int C, int& G, int& NV) {
  const int per32 = (C / 8 + 31) / 32;  // vectors per lane with one warp per row
  if (per32 > 32) return false;
  G = per32 <= 4 ? 1 : (per32 <= 8 ? 2 : (per32 <= 16 ? 4 : 8));
  NV = (per32 + G - 1) / G;
  if (G > 1 && NV < 3) NV = 3;  // only NV 3 and 4 are built for the multi-warp forms
  return true;
}

static inline int norm_stream_mode() {
  static int mode = -1;
  if (mode < 0) {
    const char* e = getenv("MOMIJO_NORM_STREAM");
    mode = (e != nullptr && e[0] == '0') ? 0 : 1;  // MOMIJO_NORM_STREAM=0 selects the row-per-CTA kernels
  }
  return mode;
}

static inline int norm_threads(int C, int vpt) {
  int nvec = C / 8;
  int t = (nvec + vpt - 1) / vpt;
  t = ((t + 31) / 32) * 32;
  return t < 32 ? 32 : t;
}

}  // namespace mmj

using namespace mmj;

#define MMJ_NORM_DISPATCH(NVv, Gv, CALL)                 \
  if (NV == NVv && G == Gv) {                            \
    constexpr int kNV = NVv, kG = Gv;                    \
    CALL;                                                \
    launched = true;                                     \
  }
#define MMJ_NORM_ALL(CALL)                                                              \
  MMJ_NORM_DISPATCH(1, 1, CALL) MMJ_NORM_DISPATCH(2, 1, CALL) MMJ_NORM_DISPATCH(3, 1, CALL) \
  MMJ_NORM_DISPATCH(4, 1, CALL) MMJ_NORM_DISPATCH(3, 2, CALL) MMJ_NORM_DISPATCH(4, 2, CALL) \
  MMJ_NORM_DISPATCH(3, 4, CALL) MMJ_NORM_DISPATCH(4, 4, CALL) MMJ_NORM_DISPATCH(3, 8, CALL) \
  MMJ_NORM_DISPATCH(4, 8, CALL)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename K>
static inline cudaError_t norm_opt_in(K kernel, int bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

// rows x C (contiguous rows), C % 8 == 0, C <= 8192. mode 0 LayerNorm, 1 RMSNorm. `status` is the
// device status word of the bounded waits (streamed kernels).
MMJ_API int mmj_norm_fwd(const void* x, const void* res, void* res_out, const void* gamma,
                         const void* beta, void* y, float* mean, float* rstd, int rows, int C,
                         float eps, int mode, int* status, void* stream) {
  if (C % 8 != 0 || C > 8 * 512 * kNormMaxVPT) return -1;
  if (rows <= 0) return 0;
  auto xs = (const __nv_bfloat16*)x;
  int G = 0, NV = 0;
  if (norm_stream_mode() && norm_split(C, G, NV) && aligned16(x) && aligned16(res) && aligned16(y) &&
      aligned16(res_out) && aligned16(gamma) && aligned16(beta)) {
    const int ntens = res != nullptr ? 2 : 1;
    NormRing ring = norm_ring(C, G, ntens, false);
    if (ring.stages >= 2) {
      const int ntiles = (rows + ring.tile_rows - 1) / ring.tile_rows;
      int dev = 0, sms = 148;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      const int grid = ntiles < sms ? ntiles : sms;
      const int smem = ring.stages * ntens * ring.tensor_bytes;
      bool launched = false;
      MMJ_NORM_ALL((norm_opt_in(norm_fwd_stream_kernel<kNV, kG>, smem),
                    launch_pdl(norm_fwd_stream_kernel<kNV, kG>, dim3(grid), dim3(kNormThreads), (size_t)smem,
                               (cudaStream_t)stream, xs, (const __nv_bfloat16*)res, (__nv_bfloat16*)res_out,
                               (const __nv_bfloat16*)gamma, (const __nv_bfloat16*)beta, (__nv_bfloat16*)y, mean,
                               rstd, rows, C, eps, mode, ring, status)))
      if (launched) return (int)cudaGetLastError();
    }
  }
  const int vpt = (C / 8 > 512) ? 2 : 1;  // at most 512 threads: the row kernels need over 64 registers
  const int threads = norm_threads(C, vpt);
  const int grid = rows;
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
                         int* status, void* stream) {
  if (C % 8 != 0 || C > 8 * 512 * kNormMaxVPT) return -1;
  if (rows <= 0) return 0;
  int G = 0, NV = 0;
  if (norm_stream_mode() && norm_split(C, G, NV) && aligned16(x) && aligned16(dy) && aligned16(dx) &&
      aligned16(dres_in) && aligned16(gamma)) {
    const int ntens = dres_in != nullptr ? 3 : 2;
    NormRing ring = norm_ring(C, G, ntens, true);
    if (ring.stages >= 2) {
      const int ntiles = (rows + ring.tile_rows - 1) / ring.tile_rows;
      int dev = 0, sms = 148;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      int grid = ntiles < sms ? ntiles : sms;
      const int cap = mmj_norm_bwd_parts(rows);  // rows of scratch the caller provided
      if (grid > cap) grid = cap;
      const int smem = ring.stages * ntens * ring.tensor_bytes;
      const bool with_beta = mode == 0 && dbeta != nullptr;
      float* sdg = scratch;
      float* sdb = with_beta ? scratch + (size_t)grid * C : nullptr;
      bool launched = false;
      if (with_beta) {
        MMJ_NORM_ALL((norm_opt_in(norm_bwd_stream_kernel<kNV, kG, true>, smem),
                      launch_pdl(norm_bwd_stream_kernel<kNV, kG, true>, dim3(grid), dim3(kNormThreads), (size_t)smem,
                                 (cudaStream_t)stream, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                 (const __nv_bfloat16*)gamma, mean, rstd, (const __nv_bfloat16*)dres_in,
                                 (__nv_bfloat16*)dx, sdg, sdb, rows, C, mode, ring, status)))
      } else {
        MMJ_NORM_ALL((norm_opt_in(norm_bwd_stream_kernel<kNV, kG, false>, smem),
                      launch_pdl(norm_bwd_stream_kernel<kNV, kG, false>, dim3(grid), dim3(kNormThreads), (size_t)smem,
                                 (cudaStream_t)stream, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                 (const __nv_bfloat16*)gamma, mean, rstd, (const __nv_bfloat16*)dres_in,
                                 (__nv_bfloat16*)dx, sdg, sdb, rows, C, mode, ring, status)))
      }
      if (launched) {
        launch_pdl(norm_bwd_finalize_kernel, dim3((C + 15) / 16), dim3(16, 64), 0, (cudaStream_t)stream,
                   (const float*)sdg, (const float*)sdb, (__nv_bfloat16*)dgamma, (__nv_bfloat16*)dbeta, grid, C,
                   accumulate);
        return (int)cudaGetLastError();
      }
    }
  }
  const int vpt = (C / 8 > 512) ? 2 : 1;  // at most 512 threads: the row kernels need over 64 registers
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
