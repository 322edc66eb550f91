// Pixel kernels for the vision package: packed HWC uint8 images resident in device memory.
//
// Every kernel is a straight restatement of the per-pixel arithmetic of the reference's CPU loops
// (nearest resize: legacy/src/momijo/vision/backend/cpu/resize_cpu.mojo:22-55; grey =
// (299 R + 587 G + 114 B) / 1000: legacy/src/momijo/vision/backend/cpu/convert_color_cpu.mojo:45;
// separable gaussian with replicated borders and a rounded uint8 intermediate:
// legacy/src/momijo/vision/transforms/filter.mojo:62-171; erode / dilate over the in-bounds part
// of the window: legacy/src/momijo/vision/transforms/morph.mojo:66-140; nearest-sample warps:
// legacy/src/momijo/vision/transforms/geom.mojo:586-640), mapped one output pixel (or a few
// bytes of one) per thread. All of them are bandwidth bound: images are read through the
// read-only path, neighbouring threads touch neighbouring bytes, and nothing is staged twice.
#include "common.cuh"

namespace mmj {

__device__ __forceinline__ int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// ---- resize ----------------------------------------------------------------------------------
__global__ void resize_nearest_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                      int ih, int iw, int c, int oh, int ow, double sy, double sx) {
  const long long n = (long long)oh * ow * c;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int ch = (int)(i % c);
    const long long p = i / c;
    const int x = (int)(p % ow), y = (int)(p / ow);
    const int yy = clampi((int)(y * sy), 0, ih - 1);
    const int xx = clampi((int)(x * sx), 0, iw - 1);
    dst[i] = __ldg(src + ((long long)yy * iw + xx) * c + ch);
  }
}

// Bilinear with pixel centres aligned ((x + 0.5) * scale - 0.5), edges clamped, round to nearest.
__global__ void resize_bilinear_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                       int ih, int iw, int c, int oh, int ow, float sy, float sx) {
  const long long n = (long long)oh * ow * c;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int ch = (int)(i % c);
    const long long p = i / c;
    const int x = (int)(p % ow), y = (int)(p / ow);
    float fy = (y + 0.5f) * sy - 0.5f, fx = (x + 0.5f) * sx - 0.5f;
    fy = fminf(fmaxf(fy, 0.f), (float)(ih - 1));
    fx = fminf(fmaxf(fx, 0.f), (float)(iw - 1));
    const int y0 = (int)fy, x0 = (int)fx;
    const int y1 = min(y0 + 1, ih - 1), x1 = min(x0 + 1, iw - 1);
    const float wy = fy - y0, wx = fx - x0;
    const float a = __ldg(src + ((long long)y0 * iw + x0) * c + ch);
    const float b = __ldg(src + ((long long)y0 * iw + x1) * c + ch);
    const float d = __ldg(src + ((long long)y1 * iw + x0) * c + ch);
    const float e = __ldg(src + ((long long)y1 * iw + x1) * c + ch);
    const float v = (a * (1.f - wx) + b * wx) * (1.f - wy) + (d * (1.f - wx) + e * wx) * wy;
    dst[i] = (uint8_t)(v + 0.5f);
  }
}

// ---- colour ----------------------------------------------------------------------------------
// order 0: channel 0 is R (RGB input); order 1: channel 0 is B (BGR input)
__global__ void to_gray_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                               long long npix, int c, int order) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < npix;
       i += (long long)gridDim.x * blockDim.x) {
    const uint8_t* px = src + i * c;
    const int c0 = __ldg(px), c1 = __ldg(px + 1), c2 = __ldg(px + 2);
    const int r = order ? c2 : c0, b = order ? c0 : c2;
    dst[i] = (uint8_t)((r * 299 + c1 * 587 + b * 114) / 1000);
  }
}

__global__ void swap_rb_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                               long long npix, int c) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < npix;
       i += (long long)gridDim.x * blockDim.x) {
    const uint8_t* px = src + i * c;
    uint8_t* q = dst + i * c;
    const uint8_t a = __ldg(px), g = __ldg(px + 1), b = __ldg(px + 2);
    q[0] = b; q[1] = g; q[2] = a;
    for (int k = 3; k < c; ++k) q[k] = __ldg(px + k);
  }
}

// ---- separable filter (gaussian): one pass along x (dir 0) or y (dir 1) ------------------------
__constant__ float c_taps[64];

__global__ void sep_filter_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int h,
                                  int w, int c, int radius, int dir) {
  const long long n = (long long)h * w * c;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int ch = (int)(i % c);
    const long long p = i / c;
    const int x = (int)(p % w), y = (int)(p / w);
    float acc = 0.f;
    for (int k = -radius; k <= radius; ++k) {
      const int xx = dir ? x : clampi(x + k, 0, w - 1);
      const int yy = dir ? clampi(y + k, 0, h - 1) : y;
      acc += c_taps[k + radius] * (float)__ldg(src + ((long long)yy * w + xx) * c + ch);
    }
    acc = fminf(fmaxf(acc, 0.f), 255.f);
    dst[i] = (uint8_t)(acc + 0.5f);
  }
}

// ---- 3x3 derivative filters on a single-channel image, replicated borders ----------------------
// mode 0: |sobel x|, 1: |sobel y|, 2: |laplacian| (4-neighbour), 3: gradient magnitude
__global__ void deriv3_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int h, int w,
                              int mode) {
  const long long n = (long long)h * w;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int x = (int)(i % w), y = (int)(i / w);
    const int xm = max(x - 1, 0), xp = min(x + 1, w - 1), ym = max(y - 1, 0), yp = min(y + 1, h - 1);
    const int a = __ldg(src + (long long)ym * w + xm), b = __ldg(src + (long long)ym * w + x),
              cc = __ldg(src + (long long)ym * w + xp), d = __ldg(src + (long long)y * w + xm),
              e = __ldg(src + (long long)y * w + x), f = __ldg(src + (long long)y * w + xp),
              g = __ldg(src + (long long)yp * w + xm), hh = __ldg(src + (long long)yp * w + x),
              k = __ldg(src + (long long)yp * w + xp);
    const int gx = (cc + 2 * f + k) - (a + 2 * d + g);
    const int gy = (g + 2 * hh + k) - (a + 2 * b + cc);
    int v;
    if (mode == 0) v = abs(gx);
    else if (mode == 1) v = abs(gy);
    else if (mode == 2) v = abs(b + d + f + hh - 4 * e);
    else v = (int)(sqrtf((float)(gx * gx + gy * gy)) + 0.5f);
    dst[i] = (uint8_t)min(v, 255);
  }
}

// ---- morphology: min (op 0) or max (op 1) over the in-bounds part of a k x k window -------------
__global__ void morph_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int h, int w,
                             int c, int radius, int op) {
  const long long n = (long long)h * w * c;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int ch = (int)(i % c);
    const long long p = i / c;
    const int x = (int)(p % w), y = (int)(p / w);
    int v = op ? 0 : 255;
    for (int yy = max(y - radius, 0); yy <= min(y + radius, h - 1); ++yy)
      for (int xx = max(x - radius, 0); xx <= min(x + radius, w - 1); ++xx) {
        const int s = __ldg(src + ((long long)yy * w + xx) * c + ch);
        v = op ? max(v, s) : min(v, s);
      }
    dst[i] = (uint8_t)v;
  }
}

// ---- warps: nearest sample at round(M^-1 [x y 1]) with a border rule ---------------------------
// border 0: constant, 1: replicate, 2: reflect (edge pixel not repeated)
__device__ __forceinline__ int border_index(int v, int n, int border, bool* inside) {
  if (v >= 0 && v < n) return v;
  if (border == 1) return clampi(v, 0, n - 1);
  if (border == 2) {
    if (n == 1) return 0;
    const int period = 2 * (n - 1);
    int m = v % period;
    if (m < 0) m += period;
    return m < n ? m : period - m;
  }
  *inside = false;
  return 0;
}

struct Mat3 { double m[9]; };

__global__ void warp_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int h, int w,
                            int c, Mat3 inv, int perspective, int border, int fill) {
  const long long n = (long long)h * w;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int x = (int)(i % w), y = (int)(i / w);
    double u = inv.m[0] * x + inv.m[1] * y + inv.m[2];
    double v = inv.m[3] * x + inv.m[4] * y + inv.m[5];
    bool inside = true;
    if (perspective) {
      const double z = inv.m[6] * x + inv.m[7] * y + inv.m[8];
      if (z == 0.0) inside = false;
      else { u /= z; v /= z; }
    }
    uint8_t* q = dst + i * c;
    if (!inside) {
      for (int k = 0; k < c; ++k) q[k] = 0;
      continue;
    }
    // round to nearest with floor (the reference truncates u + 0.5 toward zero, which would pull
    // source position -1 onto pixel 0)
    const int sx = border_index((int)floor(u + 0.5), w, border, &inside);
    const int sy = border_index((int)floor(v + 0.5), h, border, &inside);
    for (int k = 0; k < c; ++k)
      q[k] = inside ? __ldg(src + ((long long)sy * w + sx) * c + k) : (uint8_t)fill;
  }
}

// ---- histogram: per-block shared-memory bins, then one global add per bin ---------------------
__global__ void hist_kernel(const uint8_t* __restrict__ src, long long n, int stride, int offset,
                            unsigned int* __restrict__ bins) {
  __shared__ unsigned int sh[256];
  for (int i = threadIdx.x; i < 256; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    atomicAdd(&sh[__ldg(src + i * stride + offset)], 1u);
  __syncthreads();
  for (int i = threadIdx.x; i < 256; i += blockDim.x)
    if (sh[i]) atomicAdd(&bins[i], sh[i]);
}

// ---- pointwise -------------------------------------------------------------------------------
__global__ void lut_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, long long n,
                           const uint8_t* __restrict__ lut) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    dst[i] = __ldg(lut + __ldg(src + i));
}

// op 0: and, 1: or, 2: not(a), 3: saturating round(a*alpha + b*beta + gamma)
__global__ void binary_kernel(const uint8_t* __restrict__ a, const uint8_t* __restrict__ b,
                              uint8_t* __restrict__ dst, long long n, int op, float alpha, float beta,
                              float gamma) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int x = __ldg(a + i), y = b ? __ldg(b + i) : 0;
    int v;
    if (op == 0) v = x & y;
    else if (op == 1) v = x | y;
    else if (op == 2) v = (~x) & 255;
    else {
      const float f = x * alpha + y * beta + gamma;
      v = (int)(fminf(fmaxf(f, 0.f), 255.f) + 0.5f);
    }
    dst[i] = (uint8_t)v;
  }
}

static inline int grid_for(long long n) {
  long long b = (n + 255) / 256;
  const long long cap = 148LL * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace mmj

using namespace mmj;

MMJ_API int mmj_vis_resize(const void* src, void* dst, int ih, int iw, int c, int oh, int ow,
                           int bilinear, void* stream) {
  if (ih <= 0 || iw <= 0 || c <= 0 || oh <= 0 || ow <= 0) return -1;
  const long long n = (long long)oh * ow * c;
  if (bilinear)
    resize_bilinear_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)src, (uint8_t*)dst, ih, iw, c, oh, ow, (float)ih / oh, (float)iw / ow);
  else
    resize_nearest_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)src, (uint8_t*)dst, ih, iw, c, oh, ow, (double)ih / oh, (double)iw / ow);
  return (int)cudaGetLastError();
}

MMJ_API int mmj_vis_to_gray(const void* src, void* dst, long long npix, int c, int bgr, void* stream) {
  if (c < 3) return -1;
  to_gray_kernel<<<grid_for(npix), 256, 0, (cudaStream_t)stream>>>((const uint8_t*)src, (uint8_t*)dst,
                                                                    npix, c, bgr);
  return (int)cudaGetLastError();
}

MMJ_API int mmj_vis_swap_rb(const void* src, void* dst, long long npix, int c, void* stream) {
  if (c < 3) return -1;
  swap_rb_kernel<<<grid_for(npix), 256, 0, (cudaStream_t)stream>>>((const uint8_t*)src, (uint8_t*)dst,
                                                                    npix, c);
  return (int)cudaGetLastError();
}

// taps: host float[2*radius+1]; dir 0 = along x, 1 = along y
MMJ_API int mmj_vis_sep_filter(const void* src, void* dst, int h, int w, int c, const float* taps,
                               int radius, int dir, void* stream) {
  if (radius < 0 || 2 * radius + 1 > 64) return -1;
  cudaError_t e = cudaMemcpyToSymbolAsync(c_taps, taps, sizeof(float) * (2 * radius + 1), 0,
                                          cudaMemcpyHostToDevice, (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  const long long n = (long long)h * w * c;
  sep_filter_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>((const uint8_t*)src, (uint8_t*)dst, h,
                                                                   w, c, radius, dir);
  return (int)cudaGetLastError();
}

MMJ_API int mmj_vis_deriv3(const void* src, void* dst, int h, int w, int mode, void* stream) {
  deriv3_kernel<<<grid_for((long long)h * w), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)src, (uint8_t*)dst, h, w, mode);
  return (int)cudaGetLastError();
}

MMJ_API int mmj_vis_morph(const void* src, void* dst, int h, int w, int c, int ksize, int dilate,
                          void* stream) {
  if (ksize < 1) return -1;
  morph_kernel<<<grid_for((long long)h * w * c), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)src, (uint8_t*)dst, h, w, c, ksize / 2, dilate);
  return (int)cudaGetLastError();
}

// inv: host double[9], the inverse map (output pixel -> source position)
MMJ_API int mmj_vis_warp(const void* src, void* dst, int h, int w, int c, const double* inv,
                         int perspective, int border, int fill, void* stream) {
  Mat3 m;
  for (int i = 0; i < 9; ++i) m.m[i] = inv[i];
  warp_kernel<<<grid_for((long long)h * w), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)src, (uint8_t*)dst, h, w, c, m, perspective, border, fill);
  return (int)cudaGetLastError();
}

// bins: device uint32[256], zeroed by the caller; counts channel `offset` of `c`-channel pixels
MMJ_API int mmj_vis_hist(const void* src, long long npix, int c, int offset, void* bins, void* stream) {
  hist_kernel<<<grid_for(npix), 256, 0, (cudaStream_t)stream>>>((const uint8_t*)src, npix, c, offset,
                                                                 (unsigned int*)bins);
  return (int)cudaGetLastError();
}

MMJ_API int mmj_vis_lut(const void* src, void* dst, long long n, const void* lut, void* stream) {
  lut_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>((const uint8_t*)src, (uint8_t*)dst, n,
                                                            (const uint8_t*)lut);
  return (int)cudaGetLastError();
}

MMJ_API int mmj_vis_binary(const void* a, const void* b, void* dst, long long n, int op, float alpha,
                           float beta, float gamma, void* stream) {
  binary_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)a, (const uint8_t*)b, (uint8_t*)dst, n, op, alpha, beta, gamma);
  return (int)cudaGetLastError();
}
