// Neighbourhood and region kernels of the vision package on packed HWC uint8 images: median filter,
// bilateral filter, Canny edge stages (gradient + non-maximum suppression, hysteresis), CLAHE (per-tile
// clipped histogram -> look-up table, bilinear blend of the four surrounding tables) and
// connected-component labelling by label propagation with pointer jumping.
//
// The reference runs all of these as host loops (legacy/src/momijo/vision/transforms/filter.mojo:193-427,
// legacy/src/momijo/vision/transforms/color.mojo:635, legacy/src/momijo/vision/transforms/
// segmentation.mojo:99-292); each kernel restates that arithmetic with one thread per output pixel and
// no atomics on the result, so outputs do not depend on scheduling.
#include "common.cuh"

namespace mmj {

static inline int vf_grid(long long n) {
  long long b = (n + 255) / 256;
  const long long cap = 148LL * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}
__device__ __forceinline__ int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// ---- median, k x k (k odd, <= 9), replicated border ---------------------------------------------------
__global__ void median_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int h, int w, int c, int k) {
  const int r = k / 2, n = k * k, mid = n / 2;
  const long long total = (long long)h * w * c;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int ch = (int)(i % c);
    const int x = (int)((i / c) % w);
    const int y = (int)(i / ((long long)c * w));
    unsigned char v[81];
    int m = 0;
    for (int dy = -r; dy <= r; ++dy) {
      const int yy = clampi(y + dy, 0, h - 1);
      for (int dx = -r; dx <= r; ++dx) {
        const int xx = clampi(x + dx, 0, w - 1);
        v[m++] = src[((long long)yy * w + xx) * c + ch];
      }
    }
    // partial selection sort up to the middle element
    for (int a = 0; a <= mid; ++a) {
      int best = a;
      for (int b = a + 1; b < n; ++b)
        if (v[b] < v[best]) best = b;
      const unsigned char t = v[a];
      v[a] = v[best];
      v[best] = t;
    }
    dst[i] = v[mid];
  }
}

// ---- bilateral: weights exp(-(sum_c |q - p|)^2 / sc2 - (dx^2 + dy^2) / ss2), replicated border ----------
__global__ void bilateral_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int h, int w, int c,
                                 int r, float sc2, float ss2) {
  const long long total = (long long)h * w;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int x = (int)(i % w), y = (int)(i / w);
    const uint8_t* p = src + i * c;
    float num[4] = {0.f, 0.f, 0.f, 0.f};
    float den = 0.f;
    for (int dy = -r; dy <= r; ++dy) {
      const int yy = clampi(y + dy, 0, h - 1);
      for (int dx = -r; dx <= r; ++dx) {
        const int xx = clampi(x + dx, 0, w - 1);
        const uint8_t* q = src + ((long long)yy * w + xx) * c;
        float diff = 0.f;
        for (int ch = 0; ch < c; ++ch) diff += fabsf((float)q[ch] - (float)p[ch]);
        const float wgt = expf(-(diff * diff) / sc2 - (float)(dx * dx + dy * dy) / ss2);
        for (int ch = 0; ch < c; ++ch) num[ch] += wgt * (float)q[ch];
        den += wgt;
      }
    }
    for (int ch = 0; ch < c; ++ch) {
      const float v = fminf(fmaxf(num[ch] / den + 0.5f, 0.f), 255.f);
      dst[i * c + ch] = (uint8_t)v;
    }
  }
}

// ---- Canny stage 1: Sobel (replicated border), L1 magnitude, non-maximum suppression along the gradient
// sector, double threshold. cls: 0 = none, 1 = weak, 2 = strong.
__device__ __forceinline__ int sobel_mag(const uint8_t* g, int h, int w, int y, int x, int* gx_out, int* gy_out) {
  auto at = [&](int yy, int xx) { return (int)g[(long long)clampi(yy, 0, h - 1) * w + clampi(xx, 0, w - 1)]; };
  const int gx = (at(y - 1, x + 1) + 2 * at(y, x + 1) + at(y + 1, x + 1)) -
                 (at(y - 1, x - 1) + 2 * at(y, x - 1) + at(y + 1, x - 1));
  const int gy = (at(y + 1, x - 1) + 2 * at(y + 1, x) + at(y + 1, x + 1)) -
                 (at(y - 1, x - 1) + 2 * at(y - 1, x) + at(y - 1, x + 1));
  if (gx_out) *gx_out = gx;
  if (gy_out) *gy_out = gy;
  return abs(gx) + abs(gy);
}
__global__ void canny_nms_kernel(const uint8_t* __restrict__ gray, uint8_t* __restrict__ cls, int h, int w, int lo,
                                 int hi) {
  const long long total = (long long)h * w;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int x = (int)(i % w), y = (int)(i / w);
    int gx, gy;
    const int mag = sobel_mag(gray, h, w, y, x, &gx, &gy);
    // angle folded into [0, 180), sectors of 45 degrees centred on 0, 45, 90, 135 (double precision: the
    // sector borders are irrational slopes, never hit exactly by integer gradients)
    double ang = atan2((double)gy, (double)gx) * 57.29577951308232 + 180.0;
    ang = fmod(ang, 180.0);
    const int sector = ((int)floor((ang + 22.5) / 45.0)) % 4;
    const int dy1[4] = {0, 1, 1, 1}, dx1[4] = {1, 1, 0, -1};
    auto m = [&](int yy, int xx) -> int {   // zero outside the image
      if (yy < 0 || yy >= h || xx < 0 || xx >= w) return 0;
      return sobel_mag(gray, h, w, yy, xx, nullptr, nullptr);
    };
    const int n1 = m(y + dy1[sector], x + dx1[sector]);
    const int n2 = m(y - dy1[sector], x - dx1[sector]);
    const int nms = (mag >= n1 && mag >= n2) ? mag : 0;
    cls[i] = (uint8_t)(nms >= hi ? 2 : (nms >= lo ? 1 : 0));
  }
}
// ---- Canny stage 2: hysteresis. One pass promotes weak pixels that touch a strong one, repeating inside a
// 32 x 32 tile (plus a one-pixel halo) in shared memory until the tile is stable; `changed` tells the host
// whether another pass over the image is needed.
__global__ void __launch_bounds__(1024) canny_hysteresis_kernel(uint8_t* __restrict__ cls, int h, int w,
                                                                int* __restrict__ changed) {
  __shared__ uint8_t t[34][34];
  __shared__ int again;
  const int x0 = blockIdx.x * 32, y0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 34 * 34; i += blockDim.x) {
    const int yy = y0 + i / 34 - 1, xx = x0 + i % 34 - 1;
    t[i / 34][i % 34] = (yy >= 0 && yy < h && xx >= 0 && xx < w) ? cls[(long long)yy * w + xx] : 0;
  }
  __syncthreads();
  const bool inside = (y0 + ty < h) && (x0 + tx < w);
  bool promoted = false;
  for (int it = 0; it < 64; ++it) {
    if (threadIdx.x == 0) again = 0;
    __syncthreads();
    if (inside && t[ty + 1][tx + 1] == 1) {
      bool s = false;
      for (int dy = 0; dy < 3; ++dy)
        for (int dx = 0; dx < 3; ++dx) s |= (t[ty + dy][tx + dx] == 2);
      if (s) {
        t[ty + 1][tx + 1] = 2;   // a race with neighbours reading this cell only delays them by one round
        promoted = true;
        again = 1;
      }
    }
    __syncthreads();
    if (!again) break;
    __syncthreads();
  }
  if (promoted) {
    cls[(long long)(y0 + ty) * w + x0 + tx] = 2;
    *changed = 1;
  }
}
__global__ void canny_finish_kernel(const uint8_t* __restrict__ cls, uint8_t* __restrict__ out, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = cls[i] == 2 ? 255 : 0;
}

// ---- CLAHE ---------------------------------------------------------------------------------------------
// One block per tile: histogram, clip at max(1, clip * size / 256), spread the excess evenly, cumulative sum
// scaled to 255 (fp32 table). Tile borders are given by ys[ty + 1], xs[tx + 1].
__global__ void __launch_bounds__(256) clahe_lut_kernel(const uint8_t* __restrict__ a, int w, const int* __restrict__ ys,
                                                        const int* __restrict__ xs, int tx_n, float clip_limit,
                                                        float* __restrict__ luts) {
  __shared__ unsigned int hist[256];
  __shared__ double cum[256];
  const int tj = blockIdx.x % tx_n, ti = blockIdx.x / tx_n;
  const int y0 = ys[ti], y1 = ys[ti + 1], x0 = xs[tj], x1 = xs[tj + 1];
  hist[threadIdx.x] = 0;
  __syncthreads();
  const int bw = x1 - x0, size = (y1 - y0) * bw;
  for (int i = threadIdx.x; i < size; i += blockDim.x)
    atomicAdd(&hist[a[(long long)(y0 + i / bw) * w + x0 + i % bw]], 1u);   // integer counts: order does not matter
  __syncthreads();
  const double limit = fmax(1.0, (double)clip_limit * size / 256.0);
  const double hv = (double)hist[threadIdx.x];
  cum[threadIdx.x] = fmax(hv - limit, 0.0);
  __syncthreads();
  // total excess (same for every thread), then the clipped histogram, then an inclusive scan
  double excess = 0.0;
  for (int i = 0; i < 256; ++i) excess += cum[i];
  __syncthreads();
  cum[threadIdx.x] = fmin(hv, limit) + excess / 256.0;
  __syncthreads();
  if (threadIdx.x == 0) {
    double s = 0.0;
    for (int i = 0; i < 256; ++i) {
      s += cum[i];
      cum[i] = s;
    }
  }
  __syncthreads();
  const double last = fmax(cum[255], 1.0);
  luts[(long long)blockIdx.x * 256 + threadIdx.x] = (float)(cum[threadIdx.x] * 255.0 / last);
}
// Per pixel: fractional tile coordinates fi[y], fj[x] (precomputed on the host like the reference does),
// bilinear blend of the four surrounding tables, + 0.5, clamp.
__global__ void clahe_apply_kernel(const uint8_t* __restrict__ a, uint8_t* __restrict__ out, int h, int w,
                                   const float* __restrict__ fi, const float* __restrict__ fj, int ty_n, int tx_n,
                                   const float* __restrict__ luts) {
  const long long total = (long long)h * w;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int x = (int)(i % w), y = (int)(i / w);
    const float fy = fi[y], fx = fj[x];
    const int i0 = (int)floorf(fy), j0 = (int)floorf(fx);
    const int i1 = min(i0 + 1, ty_n - 1), j1 = min(j0 + 1, tx_n - 1);
    const float wy = fy - (float)i0, wx = fx - (float)j0;
    const int v = a[i];
    auto g = [&](int ii, int jj) { return luts[((long long)ii * tx_n + jj) * 256 + v]; };
    const float r = (g(i0, j0) * (1.f - wx) + g(i0, j1) * wx) * (1.f - wy) +
                    (g(i1, j0) * (1.f - wx) + g(i1, j1) * wx) * wy;
    out[i] = (uint8_t)fminf(fmaxf(r + 0.5f, 0.f), 255.f);
  }
}

// ---- connected components ------------------------------------------------------------------------------
// labels: int32 [h * w]; foreground pixels start with their own index + 1, background 0. Each pass gives a
// pixel the smallest label among itself and its neighbours, followed to its root (label l points at pixel
// l - 1); passes repeat until nothing changes. Every component ends with the (index + 1) of its first pixel
// in row-major order, whatever the scheduling.
__global__ void cc_init_kernel(const uint8_t* __restrict__ bw, int stride, int* __restrict__ labels, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    labels[i] = bw[i * stride] != 0 ? (int)(i + 1) : 0;
}
__global__ void cc_pass_kernel(int* __restrict__ labels, int h, int w, int conn8, int* __restrict__ changed) {
  const long long total = (long long)h * w;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int me = labels[i];
    if (me == 0) continue;
    const int x = (int)(i % w), y = (int)(i / w);
    int best = me;
    for (int dy = -1; dy <= 1; ++dy)
      for (int dx = -1; dx <= 1; ++dx) {
        if ((dx == 0 && dy == 0) || (!conn8 && dx != 0 && dy != 0)) continue;
        const int yy = y + dy, xx = x + dx;
        if (yy < 0 || yy >= h || xx < 0 || xx >= w) continue;
        const int l = labels[(long long)yy * w + xx];
        if (l != 0 && l < best) best = l;
      }
    // follow the chain of smaller labels to its current root
    for (int hops = 0; hops < 64; ++hops) {
      const int up = labels[best - 1];
      if (up >= best || up == 0) break;
      best = up;
    }
    if (best < me) {
      atomicMin(&labels[i], best);   // min is order independent: the fixed point does not depend on timing
      *changed = 1;
    }
  }
}

}  // namespace mmj

using namespace mmj;
#define STREAM ((cudaStream_t)stream)

MMJ_API int mmj_vis_median(const void* src, void* dst, int h, int w, int c, int ksize, void* stream) {
  if (h <= 0 || w <= 0 || c <= 0 || ksize < 1 || ksize > 9 || !(ksize & 1)) return -1;
  median_kernel<<<vf_grid((long long)h * w * c), 256, 0, STREAM>>>((const uint8_t*)src, (uint8_t*)dst, h, w, c, ksize);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_vis_bilateral(const void* src, void* dst, int h, int w, int c, int radius, float sc2, float ss2,
                              void* stream) {
  if (h <= 0 || w <= 0 || c <= 0 || c > 4 || radius < 0) return -1;
  bilateral_kernel<<<vf_grid((long long)h * w), 256, 0, STREAM>>>((const uint8_t*)src, (uint8_t*)dst, h, w, c, radius,
                                                                  sc2, ss2);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_vis_canny_nms(const void* gray, void* cls, int h, int w, int lo, int hi, void* stream) {
  if (h <= 0 || w <= 0) return -1;
  canny_nms_kernel<<<vf_grid((long long)h * w), 256, 0, STREAM>>>((const uint8_t*)gray, (uint8_t*)cls, h, w, lo, hi);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_vis_canny_hysteresis(void* cls, int h, int w, int* changed, void* stream) {
  dim3 grid((w + 31) / 32, (h + 31) / 32);
  canny_hysteresis_kernel<<<grid, 1024, 0, STREAM>>>((uint8_t*)cls, h, w, changed);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_vis_canny_finish(const void* cls, void* out, long long n, void* stream) {
  canny_finish_kernel<<<vf_grid(n), 256, 0, STREAM>>>((const uint8_t*)cls, (uint8_t*)out, n);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_vis_clahe_luts(const void* plane, int w, const int* ys, const int* xs, int ty_n, int tx_n,
                               float clip_limit, float* luts, void* stream) {
  if (ty_n <= 0 || tx_n <= 0) return -1;
  clahe_lut_kernel<<<ty_n * tx_n, 256, 0, STREAM>>>((const uint8_t*)plane, w, ys, xs, tx_n, clip_limit, luts);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_vis_clahe_apply(const void* plane, void* out, int h, int w, const float* fi, const float* fj,
                                int ty_n, int tx_n, const float* luts, void* stream) {
  clahe_apply_kernel<<<vf_grid((long long)h * w), 256, 0, STREAM>>>((const uint8_t*)plane, (uint8_t*)out, h, w, fi, fj,
                                                                    ty_n, tx_n, luts);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_vis_cc_init(const void* bw, int stride, int* labels, long long n, void* stream) {
  cc_init_kernel<<<vf_grid(n), 256, 0, STREAM>>>((const uint8_t*)bw, stride, labels, n);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_vis_cc_pass(int* labels, int h, int w, int conn8, int* changed, void* stream) {
  cc_pass_kernel<<<vf_grid((long long)h * w), 256, 0, STREAM>>>(labels, h, w, conn8, changed);
  return (int)cudaGetLastError();
}
