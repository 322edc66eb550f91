// Convolution and pooling kernels (NCHW): im2col / col2im for the GEMM-lowered convolution, direct
// fp32 convolution forward / input gradient / weight gradient / bias gradient (groups supported, so
// depthwise convolutions run here too), transposed convolution through the same kernels, max pooling
// with saved arg-max positions and average pooling, each with a deterministic backward.
//
// The reference has a one-thread-per-output max-pool and direct-convolution forward on the device
// (legacy/src/momijo/tensor/gpu/runtime.mojo:122-200) and host loops for the rest; its max-pool
// backward adds `gy` at the arg-max with a plain `+=`, which races when windows overlap
// (legacy/src/momijo/learn/nn/conv.mojo:342-405). Every backward here is written in gather form:
// one thread owns one gradient element and sums the contributions that reach it in a fixed order,
// so there are no atomics and results are bitwise reproducible.
#include "common.cuh"

namespace mmj {

struct ConvGeom {
  int N, C, H, W;        // input
  int OC, kH, kW;        // filters
  int OH, OW;            // output
  int sh, sw, ph, pw, dh, dw;
  int groups;
};

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

// ---- im2col: cols[(n, oh, ow), c * kH * kW + kh * kW + kw], row pitch ldc >= C*kH*kW (pad columns = 0) ----
template <typename T>
__global__ void im2col_kernel(const T* __restrict__ x, T* __restrict__ cols, ConvGeom g, long long ldc) {
  const long long K = (long long)g.C * g.kH * g.kW;
  const long long rows = (long long)g.N * g.OH * g.OW;
  const long long total = rows * ldc;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / ldc;
    const long long k = i - r * ldc;
    T v = from_f<T>(0.f);
    if (k < K) {
      const int kw = (int)(k % g.kW);
      const int kh = (int)((k / g.kW) % g.kH);
      const int c = (int)(k / ((long long)g.kW * g.kH));
      const int ow = (int)(r % g.OW);
      const int oh = (int)((r / g.OW) % g.OH);
      const int n = (int)(r / ((long long)g.OW * g.OH));
      const int h = oh * g.sh - g.ph + kh * g.dh;
      const int w = ow * g.sw - g.pw + kw * g.dw;
      if (h >= 0 && h < g.H && w >= 0 && w < g.W)
        v = x[(((long long)n * g.C + c) * g.H + h) * g.W + w];
    }
    cols[i] = v;
  }
}

// ---- col2im (gather form): dx[n, c, h, w] = sum over the window positions that read this element ----
template <typename T>
__global__ void col2im_kernel(const T* __restrict__ cols, T* __restrict__ dx, ConvGeom g, long long ldc) {
  const long long total = (long long)g.N * g.C * g.H * g.W;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int w = (int)(i % g.W);
    const int h = (int)((i / g.W) % g.H);
    const int c = (int)((i / ((long long)g.W * g.H)) % g.C);
    const int n = (int)(i / ((long long)g.W * g.H * g.C));
    float acc = 0.f;
    for (int kh = 0; kh < g.kH; ++kh) {
      const int hh = h + g.ph - kh * g.dh;
      if (hh < 0 || hh % g.sh) continue;
      const int oh = hh / g.sh;
      if (oh >= g.OH) continue;
      for (int kw = 0; kw < g.kW; ++kw) {
        const int ww = w + g.pw - kw * g.dw;
        if (ww < 0 || ww % g.sw) continue;
        const int ow = ww / g.sw;
        if (ow >= g.OW) continue;
        const long long r = ((long long)n * g.OH + oh) * g.OW + ow;
        acc += to_f<T>(cols[r * ldc + ((long long)c * g.kH + kh) * g.kW + kw]);
      }
    }
    dx[i] = from_f<T>(acc);
  }
}

// ---- direct convolution, fp32 accumulate; weight [OC, C/groups, kH, kW] --------------------------------
template <typename T>
__global__ void conv2d_fwd_kernel(const T* __restrict__ x, const T* __restrict__ wt, const T* __restrict__ bias,
                                  T* __restrict__ y, ConvGeom g) {
  const int cg = g.C / g.groups, ocg = g.OC / g.groups;
  const long long total = (long long)g.N * g.OC * g.OH * g.OW;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int ow = (int)(i % g.OW);
    const int oh = (int)((i / g.OW) % g.OH);
    const int oc = (int)((i / ((long long)g.OW * g.OH)) % g.OC);
    const int n = (int)(i / ((long long)g.OW * g.OH * g.OC));
    const int c0 = (oc / ocg) * cg;
    float acc = (bias != nullptr) ? to_f<T>(bias[oc]) : 0.f;
    for (int c = 0; c < cg; ++c) {
      const T* xp = x + ((long long)n * g.C + c0 + c) * g.H * g.W;
      const T* wp = wt + ((long long)oc * cg + c) * g.kH * g.kW;
      for (int kh = 0; kh < g.kH; ++kh) {
        const int h = oh * g.sh - g.ph + kh * g.dh;
        if (h < 0 || h >= g.H) continue;
        for (int kw = 0; kw < g.kW; ++kw) {
          const int w = ow * g.sw - g.pw + kw * g.dw;
          if (w < 0 || w >= g.W) continue;
          acc = fmaf(to_f<T>(xp[(long long)h * g.W + w]), to_f<T>(wp[kh * g.kW + kw]), acc);
        }
      }
    }
    y[i] = from_f<T>(acc);
  }
}

// dx[n, c, h, w] = sum_{oc in group, kh, kw} dy[n, oc, oh, ow] * wt[oc, c - c0, kh, kw]  (gather form).
// Run on (x = input of a transposed convolution, weight [Cin, Cout/groups, kH, kW]) this is also the
// forward pass of the transposed convolution; `bias` (per output channel here = per c) is added then.
template <typename T>
__global__ void conv2d_dx_kernel(const T* __restrict__ dy, const T* __restrict__ wt, const T* __restrict__ bias,
                                 T* __restrict__ dx, ConvGeom g) {
  const int cg = g.C / g.groups, ocg = g.OC / g.groups;
  const long long total = (long long)g.N * g.C * g.H * g.W;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int w = (int)(i % g.W);
    const int h = (int)((i / g.W) % g.H);
    const int c = (int)((i / ((long long)g.W * g.H)) % g.C);
    const int n = (int)(i / ((long long)g.W * g.H * g.C));
    const int grp = c / cg, cl = c - grp * cg;
    float acc = (bias != nullptr) ? to_f<T>(bias[c]) : 0.f;
    for (int o = 0; o < ocg; ++o) {
      const int oc = grp * ocg + o;
      const T* dyp = dy + ((long long)n * g.OC + oc) * g.OH * g.OW;
      const T* wp = wt + ((long long)oc * cg + cl) * g.kH * g.kW;
      for (int kh = 0; kh < g.kH; ++kh) {
        const int hh = h + g.ph - kh * g.dh;
        if (hh < 0 || hh % g.sh) continue;
        const int oh = hh / g.sh;
        if (oh >= g.OH) continue;
        for (int kw = 0; kw < g.kW; ++kw) {
          const int ww = w + g.pw - kw * g.dw;
          if (ww < 0 || ww % g.sw) continue;
          const int ow = ww / g.sw;
          if (ow >= g.OW) continue;
          acc = fmaf(to_f<T>(dyp[(long long)oh * g.OW + ow]), to_f<T>(wp[kh * g.kW + kw]), acc);
        }
      }
    }
    dx[i] = from_f<T>(acc);
  }
}

__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float x = (lane < 8) ? red[lane] : 0.f;
  x = warp_sum(x);
  __syncthreads();
  return x;
}

// dw[oc, cl, kh, kw] = sum_{n, oh, ow} dy[n, oc, oh, ow] * x[n, c0 + cl, h, w]: one block per weight
// element, threads stride over (n, oh, ow), fixed-order block reduction.
template <typename T>
__global__ void __launch_bounds__(256) conv2d_dw_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                        T* __restrict__ dwt, ConvGeom g) {
  __shared__ float red[8];
  const int cg = g.C / g.groups, ocg = g.OC / g.groups;
  const long long e = blockIdx.x;
  const int kw = (int)(e % g.kW);
  const int kh = (int)((e / g.kW) % g.kH);
  const int cl = (int)((e / ((long long)g.kW * g.kH)) % cg);
  const int oc = (int)(e / ((long long)g.kW * g.kH * cg));
  const int c = (oc / ocg) * cg + cl;
  const long long spatial = (long long)g.OH * g.OW;
  const long long total = (long long)g.N * spatial;
  float acc = 0.f;
  for (long long i = threadIdx.x; i < total; i += blockDim.x) {
    const int ow = (int)(i % g.OW);
    const int oh = (int)((i / g.OW) % g.OH);
    const int n = (int)(i / spatial);
    const int h = oh * g.sh - g.ph + kh * g.dh;
    const int w = ow * g.sw - g.pw + kw * g.dw;
    if (h < 0 || h >= g.H || w < 0 || w >= g.W) continue;
    acc = fmaf(to_f<T>(dy[((long long)n * g.OC + oc) * spatial + (long long)oh * g.OW + ow]),
               to_f<T>(x[(((long long)n * g.C + c) * g.H + h) * g.W + w]), acc);
  }
  acc = block_sum_256(acc, red);
  if (threadIdx.x == 0) dwt[e] = from_f<T>(acc);
}

// db[oc] = sum_{n, oh, ow} dy[n, oc, oh, ow]
template <typename T>
__global__ void __launch_bounds__(256) channel_sum_kernel(const T* __restrict__ dy, T* __restrict__ db, int N,
                                                          int OC, long long spatial) {
  __shared__ float red[8];
  const int oc = blockIdx.x;
  float acc = 0.f;
  for (long long i = threadIdx.x; i < (long long)N * spatial; i += blockDim.x) {
    const long long n = i / spatial, s = i - n * spatial;
    acc += to_f<T>(dy[(n * OC + oc) * spatial + s]);
  }
  acc = block_sum_256(acc, red);
  if (threadIdx.x == 0) db[oc] = from_f<T>(acc);
}

// ---- pooling ----------------------------------------------------------------------------------------------
struct PoolGeom {
  int NC, H, W, OH, OW, kH, kW, sh, sw, ph, pw;
  int count_include_pad;
};

// idx[i] = flat position (h * W + w) of the maximum inside the plane; the first maximum wins (NaN wins
// over numbers, as in the usual definition).
template <typename T>
__global__ void maxpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int* __restrict__ idx, PoolGeom g) {
  const long long total = (long long)g.NC * g.OH * g.OW;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int ow = (int)(i % g.OW);
    const int oh = (int)((i / g.OW) % g.OH);
    const long long nc = i / ((long long)g.OW * g.OH);
    const T* xp = x + nc * g.H * g.W;
    float best = -INFINITY;
    int bi = -1;
    for (int kh = 0; kh < g.kH; ++kh) {
      const int h = oh * g.sh - g.ph + kh;
      if (h < 0 || h >= g.H) continue;
      for (int kw = 0; kw < g.kW; ++kw) {
        const int w = ow * g.sw - g.pw + kw;
        if (w < 0 || w >= g.W) continue;
        const float v = to_f<T>(xp[h * g.W + w]);
        if (bi < 0 || v > best || v != v) {
          if (!(best != best)) {  // keep an earlier NaN
            best = v;
            bi = h * g.W + w;
          }
        }
      }
    }
    y[i] = from_f<T>(best);
    if (idx != nullptr) idx[i] = bi;
  }
}

// dx[nc, h, w] = sum of dy over the windows whose arg-max is (h, w): every input element looks at the
// windows that contain it (gather), so overlapping windows need no atomics.
template <typename T>
__global__ void maxpool_bwd_kernel(const T* __restrict__ dy, const int* __restrict__ idx, T* __restrict__ dx,
                                   PoolGeom g) {
  const long long total = (long long)g.NC * g.H * g.W;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int w = (int)(i % g.W);
    const int h = (int)((i / g.W) % g.H);
    const long long nc = i / ((long long)g.W * g.H);
    const int me = h * g.W + w;
    // windows (oh, ow) with oh*sh - ph <= h < oh*sh - ph + kH
    const int oh_lo = max(0, (h + g.ph - g.kH + g.sh) / g.sh), oh_hi = min(g.OH - 1, (h + g.ph) / g.sh);
    const int ow_lo = max(0, (w + g.pw - g.kW + g.sw) / g.sw), ow_hi = min(g.OW - 1, (w + g.pw) / g.sw);
    float acc = 0.f;
    for (int oh = oh_lo; oh <= oh_hi; ++oh)
      for (int ow = ow_lo; ow <= ow_hi; ++ow) {
        const long long o = (nc * g.OH + oh) * g.OW + ow;
        if (idx[o] == me) acc += to_f<T>(dy[o]);
      }
    dx[i] = from_f<T>(acc);
  }
}

__device__ __forceinline__ int pool_count(const PoolGeom& g, int oh, int ow) {
  if (g.count_include_pad) return g.kH * g.kW;
  const int h0 = max(0, oh * g.sh - g.ph), h1 = min(g.H, oh * g.sh - g.ph + g.kH);
  const int w0 = max(0, ow * g.sw - g.pw), w1 = min(g.W, ow * g.sw - g.pw + g.kW);
  return max(1, (h1 - h0) * (w1 - w0));
}

template <typename T>
__global__ void avgpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, PoolGeom g) {
  const long long total = (long long)g.NC * g.OH * g.OW;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int ow = (int)(i % g.OW);
    const int oh = (int)((i / g.OW) % g.OH);
    const long long nc = i / ((long long)g.OW * g.OH);
    const T* xp = x + nc * g.H * g.W;
    float acc = 0.f;
    for (int kh = 0; kh < g.kH; ++kh) {
      const int h = oh * g.sh - g.ph + kh;
      if (h < 0 || h >= g.H) continue;
      for (int kw = 0; kw < g.kW; ++kw) {
        const int w = ow * g.sw - g.pw + kw;
        if (w < 0 || w >= g.W) continue;
        acc += to_f<T>(xp[h * g.W + w]);
      }
    }
    y[i] = from_f<T>(acc / (float)pool_count(g, oh, ow));
  }
}

template <typename T>
__global__ void avgpool_bwd_kernel(const T* __restrict__ dy, T* __restrict__ dx, PoolGeom g) {
  const long long total = (long long)g.NC * g.H * g.W;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int w = (int)(i % g.W);
    const int h = (int)((i / g.W) % g.H);
    const long long nc = i / ((long long)g.W * g.H);
    const int oh_lo = max(0, (h + g.ph - g.kH + g.sh) / g.sh), oh_hi = min(g.OH - 1, (h + g.ph) / g.sh);
    const int ow_lo = max(0, (w + g.pw - g.kW + g.sw) / g.sw), ow_hi = min(g.OW - 1, (w + g.pw) / g.sw);
    float acc = 0.f;
    for (int oh = oh_lo; oh <= oh_hi; ++oh)
      for (int ow = ow_lo; ow <= ow_hi; ++ow)
        acc += to_f<T>(dy[(nc * g.OH + oh) * g.OW + ow]) / (float)pool_count(g, oh, ow);
    dx[i] = from_f<T>(acc);
  }
}

static inline int grid_1d(long long n) {
  long long b = (n + 255) / 256;
  if (b > 148 * 16) b = 148 * 16;
  return b < 1 ? 1 : (int)b;
}

static inline ConvGeom make_geom(const int* g) {
  ConvGeom c;
  c.N = g[0]; c.C = g[1]; c.H = g[2]; c.W = g[3]; c.OC = g[4]; c.kH = g[5]; c.kW = g[6]; c.OH = g[7]; c.OW = g[8];
  c.sh = g[9]; c.sw = g[10]; c.ph = g[11]; c.pw = g[12]; c.dh = g[13]; c.dw = g[14]; c.groups = g[15];
  return c;
}

static inline bool geom_ok(const ConvGeom& c) {
  return c.N > 0 && c.C > 0 && c.OC > 0 && c.groups > 0 && c.C % c.groups == 0 && c.OC % c.groups == 0 &&
         c.sh > 0 && c.sw > 0 && c.dh > 0 && c.dw > 0 && c.kH > 0 && c.kW > 0 && c.OH > 0 && c.OW > 0;
}

}  // namespace mmj

using namespace mmj;
#define STREAM ((cudaStream_t)stream)
#define DISPATCH(dtype, CALL_F32, CALL_BF16) \
  do {                                       \
    if ((dtype) == 1) { CALL_F32; }          \
    else if ((dtype) == 0) { CALL_BF16; }    \
    else return -1;                          \
  } while (0)

// geom: host int[16] = N, C, H, W, OC, kH, kW, OH, OW, sh, sw, ph, pw, dh, dw, groups. dtype: 0 bf16, 1 fp32.
MMJ_API int mmj_im2col(const void* x, void* cols, const int* geom, long long ldc, int dtype, void* stream) {
  const ConvGeom g = make_geom(geom);
  if (!geom_ok(g) || ldc < (long long)g.C * g.kH * g.kW) return -2;
  const long long total = (long long)g.N * g.OH * g.OW * ldc;
  DISPATCH(dtype, (im2col_kernel<float><<<grid_1d(total), 256, 0, STREAM>>>((const float*)x, (float*)cols, g, ldc)),
           (im2col_kernel<__nv_bfloat16><<<grid_1d(total), 256, 0, STREAM>>>((const __nv_bfloat16*)x,
                                                                              (__nv_bfloat16*)cols, g, ldc)));
  return (int)cudaGetLastError();
}
MMJ_API int mmj_col2im(const void* cols, void* dx, const int* geom, long long ldc, int dtype, void* stream) {
  const ConvGeom g = make_geom(geom);
  if (!geom_ok(g) || ldc < (long long)g.C * g.kH * g.kW) return -2;
  const long long total = (long long)g.N * g.C * g.H * g.W;
  DISPATCH(dtype, (col2im_kernel<float><<<grid_1d(total), 256, 0, STREAM>>>((const float*)cols, (float*)dx, g, ldc)),
           (col2im_kernel<__nv_bfloat16><<<grid_1d(total), 256, 0, STREAM>>>((const __nv_bfloat16*)cols,
                                                                              (__nv_bfloat16*)dx, g, ldc)));
  return (int)cudaGetLastError();
}
MMJ_API int mmj_conv2d_fwd(const void* x, const void* w, const void* bias, void* y, const int* geom, int dtype,
                           void* stream) {
  const ConvGeom g = make_geom(geom);
  if (!geom_ok(g)) return -2;
  const long long total = (long long)g.N * g.OC * g.OH * g.OW;
  DISPATCH(dtype, (conv2d_fwd_kernel<float><<<grid_1d(total), 256, 0, STREAM>>>((const float*)x, (const float*)w,
                                                                                 (const float*)bias, (float*)y, g)),
           (conv2d_fwd_kernel<__nv_bfloat16><<<grid_1d(total), 256, 0, STREAM>>>(
               (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, (__nv_bfloat16*)y, g)));
  return (int)cudaGetLastError();
}
MMJ_API int mmj_conv2d_dx(const void* dy, const void* w, const void* bias, void* dx, const int* geom, int dtype,
                          void* stream) {
  const ConvGeom g = make_geom(geom);
  if (!geom_ok(g)) return -2;
  const long long total = (long long)g.N * g.C * g.H * g.W;
  DISPATCH(dtype, (conv2d_dx_kernel<float><<<grid_1d(total), 256, 0, STREAM>>>((const float*)dy, (const float*)w,
                                                                                (const float*)bias, (float*)dx, g)),
           (conv2d_dx_kernel<__nv_bfloat16><<<grid_1d(total), 256, 0, STREAM>>>(
               (const __nv_bfloat16*)dy, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, (__nv_bfloat16*)dx, g)));
  return (int)cudaGetLastError();
}
MMJ_API int mmj_conv2d_dw(const void* x, const void* dy, void* dw, const int* geom, int dtype, void* stream) {
  const ConvGeom g = make_geom(geom);
  if (!geom_ok(g)) return -2;
  const long long elems = (long long)g.OC * (g.C / g.groups) * g.kH * g.kW;
  if (elems > 0x7fffffffLL) return -3;
  DISPATCH(dtype, (conv2d_dw_kernel<float><<<(unsigned)elems, 256, 0, STREAM>>>((const float*)x, (const float*)dy,
                                                                                 (float*)dw, g)),
           (conv2d_dw_kernel<__nv_bfloat16><<<(unsigned)elems, 256, 0, STREAM>>>(
               (const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dw, g)));
  return (int)cudaGetLastError();
}
MMJ_API int mmj_channel_sum(const void* dy, void* db, int N, int OC, long long spatial, int dtype, void* stream) {
  if (N <= 0 || OC <= 0 || spatial <= 0) return -2;
  DISPATCH(dtype, (channel_sum_kernel<float><<<OC, 256, 0, STREAM>>>((const float*)dy, (float*)db, N, OC, spatial)),
           (channel_sum_kernel<__nv_bfloat16><<<OC, 256, 0, STREAM>>>((const __nv_bfloat16*)dy, (__nv_bfloat16*)db, N,
                                                                       OC, spatial)));
  return (int)cudaGetLastError();
}

// pool geom: host int[12] = NC, H, W, OH, OW, kH, kW, sh, sw, ph, pw, count_include_pad
static inline PoolGeom make_pool(const int* g) {
  PoolGeom p;
  p.NC = g[0]; p.H = g[1]; p.W = g[2]; p.OH = g[3]; p.OW = g[4]; p.kH = g[5]; p.kW = g[6]; p.sh = g[7]; p.sw = g[8];
  p.ph = g[9]; p.pw = g[10]; p.count_include_pad = g[11];
  return p;
}
static inline bool pool_ok(const PoolGeom& p) {
  return p.NC > 0 && p.H > 0 && p.W > 0 && p.OH > 0 && p.OW > 0 && p.kH > 0 && p.kW > 0 && p.sh > 0 && p.sw > 0 &&
         (long long)p.H * p.W < 0x7fffffffLL;
}
MMJ_API int mmj_maxpool2d_fwd(const void* x, void* y, int* idx, const int* geom, int dtype, void* stream) {
  const PoolGeom g = make_pool(geom);
  if (!pool_ok(g)) return -2;
  const long long total = (long long)g.NC * g.OH * g.OW;
  DISPATCH(dtype, (maxpool_fwd_kernel<float><<<grid_1d(total), 256, 0, STREAM>>>((const float*)x, (float*)y, idx, g)),
           (maxpool_fwd_kernel<__nv_bfloat16><<<grid_1d(total), 256, 0, STREAM>>>((const __nv_bfloat16*)x,
                                                                                   (__nv_bfloat16*)y, idx, g)));
  return (int)cudaGetLastError();
}
MMJ_API int mmj_maxpool2d_bwd(const void* dy, const int* idx, void* dx, const int* geom, int dtype, void* stream) {
  const PoolGeom g = make_pool(geom);
  if (!pool_ok(g)) return -2;
  const long long total = (long long)g.NC * g.H * g.W;
  DISPATCH(dtype, (maxpool_bwd_kernel<float><<<grid_1d(total), 256, 0, STREAM>>>((const float*)dy, idx, (float*)dx, g)),
           (maxpool_bwd_kernel<__nv_bfloat16><<<grid_1d(total), 256, 0, STREAM>>>((const __nv_bfloat16*)dy, idx,
                                                                                   (__nv_bfloat16*)dx, g)));
  return (int)cudaGetLastError();
}
MMJ_API int mmj_avgpool2d_fwd(const void* x, void* y, const int* geom, int dtype, void* stream) {
  const PoolGeom g = make_pool(geom);
  if (!pool_ok(g)) return -2;
  const long long total = (long long)g.NC * g.OH * g.OW;
  DISPATCH(dtype, (avgpool_fwd_kernel<float><<<grid_1d(total), 256, 0, STREAM>>>((const float*)x, (float*)y, g)),
           (avgpool_fwd_kernel<__nv_bfloat16><<<grid_1d(total), 256, 0, STREAM>>>((const __nv_bfloat16*)x,
                                                                                   (__nv_bfloat16*)y, g)));
  return (int)cudaGetLastError();
}
MMJ_API int mmj_avgpool2d_bwd(const void* dy, void* dx, const int* geom, int dtype, void* stream) {
  const PoolGeom g = make_pool(geom);
  if (!pool_ok(g)) return -2;
  const long long total = (long long)g.NC * g.H * g.W;
  DISPATCH(dtype, (avgpool_bwd_kernel<float><<<grid_1d(total), 256, 0, STREAM>>>((const float*)dy, (float*)dx, g)),
           (avgpool_bwd_kernel<__nv_bfloat16><<<grid_1d(total), 256, 0, STREAM>>>((const __nv_bfloat16*)dy,
                                                                                   (__nv_bfloat16*)dx, g)));
  return (int)cudaGetLastError();
}
