// Bandwidth-bound kernels: activations (GELU, SiLU/SwiGLU, ReLU family), RoPE, embedding
// gather / scatter-add, column sums (bias gradients), casts, fills, transposes, one-hot,
// where, stateless-hash dropout and the NCHW packers.
//
// All bf16 kernels move 16 bytes per thread per access. They stand in for the reference's
// scalar Mojo GPU kernels (legacy/src/momijo/tensor/gpu/runtime.mojo:1027-1040 transpose,
// :1367-1634 layout packers, :1958-1970 one-hot, :2125-2132 copy; legacy/src/momijo/tensor/
// device.mojo:203-236 fills) and CPU-emulated launchers (runtime.mojo:916-991 where/dropout).
#include "common.cuh"

namespace mmj {

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 q = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z),
         d = unpack_bf16x2(q.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 q;
  q.x = pack_bf16x2(f[0], f[1]);
  q.y = pack_bf16x2(f[2], f[3]);
  q.z = pack_bf16x2(f[4], f[5]);
  q.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = q;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }
__device__ __forceinline__ float silu_grad_f(float x) {
  float s = 1.0f / (1.0f + __expf(-x));
  return s * (1.0f + x * (1.0f - s));
}

// ---- unary activations -----------------------------------------------------------------
// op: 0 gelu(tanh), 1 silu, 2 relu, 3 leaky_relu(alpha), 4 sigmoid, 5 tanh
__device__ __forceinline__ float act_fwd(float x, int op, float alpha) {
  switch (op) {
    case 0: return gelu_tanh(x);
    case 1: return silu_f(x);
    case 2: return fmaxf(x, 0.f);
    case 3: return x > 0.f ? x : alpha * x;
    case 4: return 1.0f / (1.0f + __expf(-x));
    default: return tanhf(x);
  }
}
__device__ __forceinline__ float act_bwd(float x, int op, float alpha) {
  switch (op) {
    case 0: return gelu_tanh_grad(x);
    case 1: return silu_grad_f(x);
    case 2: return x > 0.f ? 1.f : 0.f;
    case 3: return x > 0.f ? 1.f : alpha;
    case 4: { float s = 1.0f / (1.0f + __expf(-x)); return s * (1.f - s); }
    default: { float t = tanhf(x); return 1.f - t * t; }
  }
}

__global__ void act_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                               long long n8, int op, float alpha) {
  pdl_wait();
  pdl_trigger();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    float f[8];
    ld8(x + i * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = act_fwd(f[j], op, alpha);
    st8(y + i * 8, f);
  }
}
__global__ void act_bwd_kernel(const __nv_bfloat16* __restrict__ x,
                               const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx,
                               long long n8, int op, float alpha) {
  pdl_wait();
  pdl_trigger();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    float f[8], g[8];
    ld8(x + i * 8, f);
    ld8(dy + i * 8, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= act_bwd(f[j], op, alpha);
    st8(dx + i * 8, g);
  }
}

// ---- SwiGLU: y = silu(gate) * up; gate/up are column halves of a [rows, 2F] matrix --------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ y,
                                  long long rows, int F) {
  pdl_wait();
  pdl_trigger();
  const int f8 = F >> 3;
  const long long total = rows * f8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / f8;
    const int c = (int)(i - r * f8) * 8;
    float g[8], u[8];
    ld8(gu + r * 2 * F + c, g);
    ld8(gu + r * 2 * F + F + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] = silu_f(g[j]) * u[j];
    st8(y + r * F + c, g);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                  const __nv_bfloat16* __restrict__ dy,
                                  __nv_bfloat16* __restrict__ dgu, long long rows, int F) {
  pdl_wait();
  pdl_trigger();
  const int f8 = F >> 3;
  const long long total = rows * f8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / f8;
    const int c = (int)(i - r * f8) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    ld8(gu + r * 2 * F + c, g);
    ld8(gu + r * 2 * F + F + c, u);
    ld8(dy + r * F + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dg[j] = d[j] * u[j] * silu_grad_f(g[j]);
      du[j] = d[j] * silu_f(g[j]);
    }
    st8(dgu + r * 2 * F + c, dg);
    st8(dgu + r * 2 * F + F + c, du);
  }
}

// ---- RoPE (half-split pairs: (x[i], x[i + D/2])) on heads laid out inside a row -------------
// x: rows x ld; heads start at column head_off + h * D for h < n_heads. pos = row % T.
// cs: [T, D/2] float2 (cos, sin). sign = +1 forward, -1 backward (inverse rotation).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float2* __restrict__ cs,
                            long long rows, long long ld, int head_off, int n_heads, int D, int T,
                            float sign) {
  pdl_wait();
  pdl_trigger();
  const int half = D >> 1;
  const int per_row = n_heads * (half >> 3);  // 8 pairs per thread
  const long long total = rows * per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row;
    const int w = (int)(i - r * per_row);
    const int h = w / (half >> 3);
    const int c = (w - h * (half >> 3)) * 8;
    const int pos = (int)(r % T);
    __nv_bfloat16* p = x + r * ld + head_off + h * D + c;
    float a[8], b[8];
    ld8(p, a);
    ld8(p + half, b);
    const float2* t = cs + (size_t)pos * half + c;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float cc = t[j].x, sn = sign * t[j].y;
      const float na = a[j] * cc - b[j] * sn;
      const float nb = b[j] * cc + a[j] * sn;
      a[j] = na; b[j] = nb;
    }
    st8(p, a);
    st8(p + half, b);
  }
}

// ---- embedding ---------------------------------------------------------------------------
// out[row] = wte[tok[row]] (+ wpe[row % T])
__global__ void embedding_fwd_kernel(const long long* __restrict__ tok,
                                     const __nv_bfloat16* __restrict__ wte,
                                     const __nv_bfloat16* __restrict__ wpe,
                                     __nv_bfloat16* __restrict__ out, long long rows, int C, int T,
                                     int vocab) {
  const int c8 = C >> 3;
  const long long total = rows * c8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / c8;
    const int c = (int)(i - r * c8) * 8;
    long long t = tok[r];
    if (!index_ok(t, vocab, /*site=*/1)) t = t < 0 ? 0 : vocab - 1;  // clamp (recorded in debug builds)
    float a[8];
    ld8(wte + t * C + c, a);
    if (wpe != nullptr) {
      float b[8];
      ld8(wpe + (r % T) * C + c, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += b[j];
    }
    st8(out + r * C + c, a);
  }
}

// dwte[tok[row]] += dout[row]  (bf16x2 atomics; rows with the same token collide rarely)
__global__ void embedding_bwd_wte_kernel(const long long* __restrict__ tok,
                                         const __nv_bfloat16* __restrict__ dout,
                                         __nv_bfloat16* __restrict__ dwte, long long rows, int C,
                                         int vocab) {
  const int c2 = C >> 1;
  const long long total = rows * c2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / c2;
    const int c = (int)(i - r * c2) * 2;
    long long t = tok[r];
    if (!index_ok(t, vocab, /*site=*/2)) continue;
    __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(dout + r * C + c);
    atomicAdd(reinterpret_cast<__nv_bfloat162*>(dwte + t * C + c), v);
  }
}

// dwpe[t] (+)= sum_b dout[b*T + t]
__global__ void embedding_bwd_wpe_kernel(const __nv_bfloat16* __restrict__ dout,
                                         __nv_bfloat16* __restrict__ dwpe, int B, int T, int C,
                                         int accumulate) {
  const int c8 = C >> 3;
  const long long total = (long long)T * c8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / c8);
    const int c = (int)(i - (long long)t * c8) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int b = 0; b < B; ++b) {
      float f[8];
      ld8(dout + ((size_t)b * T + t) * C + c, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    if (accumulate) {
      float f[8];
      ld8(dwpe + (size_t)t * C + c, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    st8(dwpe + (size_t)t * C + c, acc);
  }
}

// ---- column sums: out[n] = sum_m x[m, n]  (bias gradients) -----------------------------------
// Stage 1: grid (ceil(N/64), S); 256 threads as 8 column groups x 32 row lanes. Each thread sums 8
// columns over its rows (a warp reads four 128-byte row pieces per load) and the block writes one
// partial row into scratch[S, N]. Narrow column strips keep several CTAs on every SM even for
// N = 768, where 256-column strips left most of the load latency exposed. Stage 2 folds the S rows.
__global__ void colsum_partial_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                      float* __restrict__ scratch, int M, int N) {
  pdl_wait();
  pdl_trigger();
  __shared__ float sm[8][64];
  const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
  const int col = (blockIdx.x * 8 + tx) * 8;
  const int S = gridDim.y;
  const int rows_per = (M + S - 1) / S;
  const int r0 = blockIdx.y * rows_per;
  const int r1 = min(M, r0 + rows_per);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col < N) {
    if (col + 8 <= N) {
#pragma unroll 4
      for (int r = r0 + ty; r < r1; r += 32) {
        float f[8];
        ld8(x + (size_t)r * ldx + col, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
    } else {
      for (int r = r0 + ty; r < r1; r += 32)
        for (int j = 0; j < 8; ++j)
          if (col + j < N) acc[j] += __bfloat162float(x[(size_t)r * ldx + col + j]);
    }
  }
  // fold the four row lanes of a warp, then the eight warps
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 8);
    acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 16);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane < 8) {
#pragma unroll
    for (int j = 0; j < 8; ++j) sm[warp][lane * 8 + j] = acc[j];
  }
  __syncthreads();
  if (threadIdx.x < 64) {
    const int c = blockIdx.x * 64 + threadIdx.x;
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += sm[w][threadIdx.x];
    if (c < N) scratch[(size_t)blockIdx.y * N + c] = t;
  }
}
// block (32, 8): 32 adjacent columns, the partial rows split over threadIdx.y
__global__ void colsum_finalize_kernel(const float* __restrict__ scratch,
                                       __nv_bfloat16* __restrict__ out_bf16,
                                       float* __restrict__ out_f32, int S, int N, int accumulate) {
  pdl_wait();
  pdl_trigger();
  __shared__ float sm[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (c < N)
    for (int p = threadIdx.y; p < S; p += 8) s += scratch[(size_t)p * N + c];
  sm[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y != 0 || c >= N) return;
  s = 0.f;
#pragma unroll
  for (int y = 0; y < 8; ++y) s += sm[y][threadIdx.x];
  if (out_bf16 != nullptr) {
    if (accumulate) s += __bfloat162float(out_bf16[c]);
    out_bf16[c] = __float2bfloat16(s);
  } else {
    if (accumulate) s += out_f32[c];
    out_f32[c] = s;
  }
}

// ---- split-K reduction: out[i] (+)= sum_s parts[s][i]  (fp32 slabs -> bf16) ---------------------
__global__ void splitk_reduce_kernel(const float* __restrict__ parts, long long slab, int S,
                                     __nv_bfloat16* __restrict__ out, long long n, int accumulate) {
  pdl_wait();
  pdl_trigger();
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 8; i < n;
       i += (long long)gridDim.x * blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < S; ++s) {
      const float4 a = *reinterpret_cast<const float4*>(parts + s * slab + i);
      const float4 b = *reinterpret_cast<const float4*>(parts + s * slab + i + 4);
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    if (accumulate) {
      float old[8];
      ld8(out + i, old);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += old[j];
    }
    st8(out + i, acc);
  }
}

// ---- in-place scaling by a device scalar, skipped when the scalar is exactly 1 -------------------
// Backward passes receive the gradient of the loss as a device scalar; it is 1 for a plain
// `loss.backward()`. Every CTA reads it first and leaves at once in that case, so the common path
// costs one empty launch and no host synchronisation; any other value scales the matrix in place.
__global__ void scale_bf16_dev_kernel(__nv_bfloat16* __restrict__ x, long long ld, long long rows,
                                      int cols, const float* __restrict__ s) {
  const float sc = *s;
  if (sc == 1.0f) return;
  const int vec_per_row = cols >> 3;  // cols % 8 == 0 and ld % 8 == 0
  const long long nvec = rows * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = (int)(i - r * vec_per_row) * 8;
    float f[8];
    ld8(x + r * ld + c, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] *= sc;
    st8(x + r * ld + c, f);
  }
}

// ---- casts, fills, axpy ------------------------------------------------------------------------
__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                        long long n) {
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < n;
       i += (long long)gridDim.x * blockDim.x * 4) {
    if (i + 4 <= n) {
      float4 v = *reinterpret_cast<const float4*>(x + i);
      uint2 q;
      q.x = pack_bf16x2(v.x, v.y);
      q.y = pack_bf16x2(v.z, v.w);
      *reinterpret_cast<uint2*>(y + i) = q;
    } else {
      for (long long j = i; j < n; ++j) y[j] = __float2bfloat16(x[j]);
    }
  }
}
__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ y,
                                        long long n) {
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < n;
       i += (long long)gridDim.x * blockDim.x * 4) {
    if (i + 4 <= n) {
      uint2 q = *reinterpret_cast<const uint2*>(x + i);
      float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y);
      *reinterpret_cast<float4*>(y + i) = make_float4(a.x, a.y, b.x, b.y);
    } else {
      for (long long j = i; j < n; ++j) y[j] = __bfloat162float(x[j]);
    }
  }
}
__global__ void fill_f32_kernel(float* __restrict__ y, float v, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    y[i] = v;
}
__global__ void fill_f64_kernel(double* __restrict__ y, double v, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    y[i] = v;
}
__global__ void fill_bf16_kernel(__nv_bfloat16* __restrict__ y, float v, long long n) {
  const __nv_bfloat16 b = __float2bfloat16(v);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    y[i] = b;
}
// y = a*x + b*y  (bf16, fp32 math)
__global__ void axpby_bf16_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                  float a, float b, long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    float f[8], g[8];
    ld8(x + i * 8, f);
    ld8(y + i * 8, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] = a * f[j] + b * g[j];
    st8(y + i * 8, g);
  }
}

// ---- 2-D transpose (tiled through shared memory; both sides coalesced) ------------------------
template <typename T>
__global__ void transpose2d_kernel(const T* __restrict__ x, T* __restrict__ y, int H, int W) {
  __shared__ T tile[32][33];
  int bx = blockIdx.x * 32, by = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int r = by + j, c = bx + threadIdx.x;
    if (r < H && c < W) tile[j][threadIdx.x] = x[(size_t)r * W + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int r = bx + j, c = by + threadIdx.x;  // output is [W, H]
    if (r < W && c < H) y[(size_t)r * H + c] = tile[threadIdx.x][j];
  }
}

// ---- one-hot, where, dropout, strided copy ------------------------------------------------------
__global__ void one_hot_f32_kernel(const long long* __restrict__ labels, float* __restrict__ out,
                                   long long n, int C) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n * C;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / C;
    const int c = (int)(i - r * C);
    out[i] = (labels[r] == c) ? 1.f : 0.f;
  }
}
__global__ void where_f32_kernel(const int* __restrict__ cond, const float* __restrict__ a,
                                 const float* __restrict__ b, float* __restrict__ out, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    out[i] = cond[i] != 0 ? a[i] : b[i];
}

// Stateless dropout: keep element i iff u01(hash(seed, i)) < 1 - p, scale kept values by
// 1/(1-p). The same seed gives the same mask on every call, which is the documented behaviour
// of the reference layer (legacy/src/momijo/learn/nn/layers.mojo:1336-1345, 1431-1455).
__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__global__ void dropout_f32_kernel(const float* __restrict__ x, float* __restrict__ y,
                                   unsigned char* __restrict__ mask, long long n, float p,
                                   unsigned long long seed) {
  const float keep = 1.f - p;
  const float scale = keep > 0.f ? 1.f / keep : 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const uint64_t h = mix64(seed ^ mix64((uint64_t)i));
    const float u = (float)(h >> 40) * (1.0f / 16777216.0f);
    const bool k = u < keep;
    y[i] = k ? x[i] * scale : 0.f;
    if (mask != nullptr) mask[i] = k ? 1 : 0;
  }
}
__global__ void dropout_bf16_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                    long long n, float p, unsigned long long seed) {
  const float keep = 1.f - p;
  const float scale = keep > 0.f ? 1.f / keep : 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const uint64_t h = mix64(seed ^ mix64((uint64_t)i));
    const float u = (float)(h >> 40) * (1.0f / 16777216.0f);
    y[i] = (u < keep) ? __float2bfloat16(__bfloat162float(x[i]) * scale) : __float2bfloat16(0.f);
  }
}

// Copy an image (HW, HWC or CHW float32) into slot n of an NCHW batch.
// layout: 0 = HW (C = 1), 1 = HWC, 2 = CHW.
__global__ void pack_nchw_kernel(const float* __restrict__ src, float* __restrict__ dst, int n,
                                 int C, int H, int W, int layout) {
  const long long total = (long long)C * H * W;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i / ((long long)H * W));
    const int hw = (int)(i - (long long)c * H * W);
    float v;
    if (layout == 1) v = src[(size_t)hw * C + c];
    else v = src[i];
    dst[(size_t)n * total + i] = v;
  }
}

// Strided 2-D cast: dst[r, c] = bf16(src[r, c]) for r < rows, c < cols (cols % 4 == 0).
__global__ void cast_f32_to_bf16_2d_kernel(const float* __restrict__ src, long long lds,
                                           __nv_bfloat16* __restrict__ dst, long long ldd,
                                           long long rows, int cols) {
  pdl_wait();
  pdl_trigger();
  const int c4 = cols >> 2;
  const long long total = rows * c4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / c4;
    const int c = (int)(i - r * c4) * 4;
    float4 v = *reinterpret_cast<const float4*>(src + r * lds + c);
    uint2 q;
    q.x = pack_bf16x2(v.x, v.y);
    q.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(dst + r * ldd + c) = q;
  }
}

static inline int grid_for(long long work, int threads) {
  long long g = (work + threads - 1) / threads;
  if (g > 148 * 16) g = 148 * 16;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace mmj

using namespace mmj;
#define STREAM ((cudaStream_t)stream)

MMJ_API int mmj_act_fwd(const void* x, void* y, long long n, int op, float alpha, void* stream) {
  if (n % 8) return -1;
  if (n == 0) return 0;
  launch_pdl(act_fwd_kernel, dim3(grid_for(n / 8, 256)), dim3(256), 0, STREAM, (const __nv_bfloat16*)x,
             (__nv_bfloat16*)y, n / 8, op, alpha);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_act_bwd(const void* x, const void* dy, void* dx, long long n, int op, float alpha,
                        void* stream) {
  if (n % 8) return -1;
  if (n == 0) return 0;
  launch_pdl(act_bwd_kernel, dim3(grid_for(n / 8, 256)), dim3(256), 0, STREAM, (const __nv_bfloat16*)x,
             (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, n / 8, op, alpha);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_swiglu_fwd(const void* gu, void* y, long long rows, int F, void* stream) {
  if (F % 8) return -1;
  if (rows == 0) return 0;
  launch_pdl(swiglu_fwd_kernel, dim3(grid_for(rows * (F / 8), 256)), dim3(256), 0, STREAM,
             (const __nv_bfloat16*)gu, (__nv_bfloat16*)y, rows, F);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_swiglu_bwd(const void* gu, const void* dy, void* dgu, long long rows, int F,
                           void* stream) {
  if (F % 8) return -1;
  if (rows == 0) return 0;
  launch_pdl(swiglu_bwd_kernel, dim3(grid_for(rows * (F / 8), 256)), dim3(256), 0, STREAM,
             (const __nv_bfloat16*)gu, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dgu, rows, F);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_rope(void* x, const void* cos_sin, long long rows, long long ld, int head_off,
                     int n_heads, int D, int T, float sign, void* stream) {
  if (D % 16 || ld % 8 || head_off % 8) return -1;
  if (rows == 0 || n_heads == 0) return 0;
  const long long work = rows * n_heads * (D / 16);
  launch_pdl(rope_kernel, dim3(grid_for(work, 256)), dim3(256), 0, STREAM, (__nv_bfloat16*)x,
             (const float2*)cos_sin, rows, ld, head_off, n_heads, D, T, sign);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_embedding_fwd(const long long* tok, const void* wte, const void* wpe, void* out,
                              long long rows, int C, int T, int vocab, void* stream) {
  if (C % 8) return -1;
  if (rows == 0) return 0;
  embedding_fwd_kernel<<<grid_for(rows * (C / 8), 256), 256, 0, STREAM>>>(
      tok, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, (__nv_bfloat16*)out, rows, C, T,
      vocab);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_embedding_bwd(const long long* tok, const void* dout, void* dwte, void* dwpe,
                              long long rows, int C, int T, int vocab, int accumulate_wpe,
                              void* stream) {
  if (C % 8) return -1;
  if (rows == 0) return 0;
  if (dwte != nullptr)
    embedding_bwd_wte_kernel<<<grid_for(rows * (C / 2), 256), 256, 0, STREAM>>>(
        tok, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dwte, rows, C, vocab);
  if (dwpe != nullptr)
    embedding_bwd_wpe_kernel<<<grid_for((long long)T * (C / 8), 128), 128, 0, STREAM>>>(
        (const __nv_bfloat16*)dout, (__nv_bfloat16*)dwpe, (int)(rows / T), T, C, accumulate_wpe);
  return (int)cudaGetLastError();
}

// Column sum with caller-provided scratch of mmj_colsum_splits(M) * N floats.
MMJ_API int mmj_colsum_splits(int M) {
  int s = (M + 255) / 256;
  if (s > 64) s = 64;
  if (s < 1) s = 1;
  return s;
}
MMJ_API int mmj_colsum_bf16(const void* x, long long ldx, void* out_bf16, float* out_f32,
                            float* scratch, int M, int N, int accumulate, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (ldx % 8) return -1;
  const int S = mmj_colsum_splits(M);
  dim3 grid((N + 63) / 64, S);
  launch_pdl(colsum_partial_kernel, grid, dim3(256), 0, STREAM, (const __nv_bfloat16*)x, ldx, scratch, M, N);
  launch_pdl(colsum_finalize_kernel, dim3((N + 31) / 32), dim3(32, 8), 0, STREAM, (const float*)scratch,
             (__nv_bfloat16*)out_bf16, out_f32, S, N, accumulate);
  return (int)cudaGetLastError();
}

// Sum S fp32 slabs of n elements (slab stride `slab`, n a multiple of 8) into a bf16 vector.
MMJ_API int mmj_splitk_reduce(const float* parts, long long slab, int S, void* out, long long n,
                              int accumulate, void* stream) {
  if (n == 0) return 0;
  if (n % 8 || slab % 4 || S < 1) return -1;
  launch_pdl(splitk_reduce_kernel, dim3(grid_for(n / 8, 256)), dim3(256), 0, STREAM, parts, slab, S,
             (__nv_bfloat16*)out, n, accumulate);
  return (int)cudaGetLastError();
}

MMJ_API int mmj_cast_f32_to_bf16(const float* x, void* y, long long n, void* stream) {
  if (n == 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_for((n + 3) / 4, 256), 256, 0, STREAM>>>(x, (__nv_bfloat16*)y, n);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_cast_bf16_to_f32(const void* x, float* y, long long n, void* stream) {
  if (n == 0) return 0;
  cast_bf16_to_f32_kernel<<<grid_for((n + 3) / 4, 256), 256, 0, STREAM>>>((const __nv_bfloat16*)x,
                                                                          y, n);
  return (int)cudaGetLastError();
}
// dtype: 0 f32, 1 f64, 2 bf16
MMJ_API int mmj_fill(void* y, double v, long long n, int dtype, void* stream) {
  if (n == 0) return 0;
  const int g = grid_for(n, 256);
  if (dtype == 0) fill_f32_kernel<<<g, 256, 0, STREAM>>>((float*)y, (float)v, n);
  else if (dtype == 1) fill_f64_kernel<<<g, 256, 0, STREAM>>>((double*)y, v, n);
  else fill_bf16_kernel<<<g, 256, 0, STREAM>>>((__nv_bfloat16*)y, (float)v, n);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_scale_bf16_dev(void* x, long long ld, long long rows, int cols, const float* s,
                               void* stream) {
  if ((cols & 7) || (ld & 7)) return -1;
  if (rows == 0 || cols == 0) return 0;
  scale_bf16_dev_kernel<<<148 * 8, 256, 0, STREAM>>>((__nv_bfloat16*)x, ld, rows, cols, s);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_axpby_bf16(const void* x, void* y, float a, float b, long long n, void* stream) {
  if (n % 8) return -1;
  if (n == 0) return 0;
  axpby_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, STREAM>>>((const __nv_bfloat16*)x,
                                                            (__nv_bfloat16*)y, a, b, n / 8);
  return (int)cudaGetLastError();
}
// elem_bytes: 2 or 4
MMJ_API int mmj_transpose2d(const void* x, void* y, int H, int W, int elem_bytes, void* stream) {
  if (H <= 0 || W <= 0) return 0;
  dim3 grid((W + 31) / 32, (H + 31) / 32), block(32, 8);
  if (elem_bytes == 4)
    transpose2d_kernel<float><<<grid, block, 0, STREAM>>>((const float*)x, (float*)y, H, W);
  else if (elem_bytes == 2)
    transpose2d_kernel<unsigned short>
        <<<grid, block, 0, STREAM>>>((const unsigned short*)x, (unsigned short*)y, H, W);
  else
    return -1;
  return (int)cudaGetLastError();
}
MMJ_API int mmj_one_hot_f32(const long long* labels, float* out, long long n, int C, void* stream) {
  if (n == 0) return 0;
  one_hot_f32_kernel<<<grid_for(n * C, 256), 256, 0, STREAM>>>(labels, out, n, C);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_where_f32(const int* cond, const float* a, const float* b, float* out, long long n,
                          void* stream) {
  if (n == 0) return 0;
  where_f32_kernel<<<grid_for(n, 256), 256, 0, STREAM>>>(cond, a, b, out, n);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_dropout_f32(const float* x, float* y, unsigned char* mask, long long n, float p,
                            unsigned long long seed, void* stream) {
  if (n == 0) return 0;
  dropout_f32_kernel<<<grid_for(n, 256), 256, 0, STREAM>>>(x, y, mask, n, p, seed);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_dropout_bf16(const void* x, void* y, long long n, float p, unsigned long long seed,
                             void* stream) {
  if (n == 0) return 0;
  dropout_bf16_kernel<<<grid_for(n, 256), 256, 0, STREAM>>>((const __nv_bfloat16*)x,
                                                            (__nv_bfloat16*)y, n, p, seed);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_pack_nchw(const float* src, float* dst, int n, int C, int H, int W, int layout,
                          void* stream) {
  const long long total = (long long)C * H * W;
  if (total == 0) return 0;
  pack_nchw_kernel<<<grid_for(total, 256), 256, 0, STREAM>>>(src, dst, n, C, H, W, layout);
  return (int)cudaGetLastError();
}
// Host-callable twin of the dropout hash so the CPU path produces the same mask.
MMJ_API unsigned long long mmj_mix64(unsigned long long z) { return mix64(z); }

// ------------------------------------------------------------------------------------------------
// Column sum without any allocation (declared in momijo_b200.h).
//
// Some callers of this library cannot allocate device memory at the point where they need a
// bias gradient: code running inside a memory-pool "no allocation" region, a serving loop that
// has handed all free memory to its KV cache, or a plugin whose host forbids cudaMalloc after
// start-up. mmj_colsum_bf16 asks such callers for `splits * N` floats of scratch; this variant
// keeps the scratch inside the library image instead, in a fixed-size device array that every
// GPU loading the library holds until the process exits (kStaticColsumFloats * 4 bytes = 4 MiB).
//
// The array's name below is only a host-side handle. Its device address is looked up once per
// device with cudaGetSymbolAddress (with that device current) during the first call on the
// device, so that first call should be made before any stream capture begins. Later calls do
// no set-up work. Nothing here calls cudaMalloc, cudaFree or any allocating routine.
//
// All calls on a device share the one array and it keeps whatever the last call left in it.
// Stage 1 overwrites every partial that stage 2 reads, so nothing needs clearing, but two calls
// that overlap on the GPU (different streams) would race on it: issue them on one stream, or
// order them with events.
// ------------------------------------------------------------------------------------------------
namespace mmj {
constexpr int kStaticColsumMaxN = 16384;
constexpr int kStaticColsumMaxSplits = 64;
constexpr long long kStaticColsumFloats = (long long)kStaticColsumMaxN * kStaticColsumMaxSplits;
constexpr int kStaticMaxDevices = 64;
static __device__ __align__(256) float g_colsum_static_scratch[kStaticColsumFloats];
static float* g_colsum_static_ptr[kStaticMaxDevices] = {nullptr};
}  // namespace mmj

// Return codes of mmj_colsum_bf16_static (0 = ok, > 0 = CUDA error code).
//   -1  leading dimension not a multiple of 8 elements
//   -20 N exceeds mmj_colsum_bf16_static_max_n()
//   -21 device ordinal outside the table kept by the library
//   -22 the device address of the built-in scratch could not be obtained
MMJ_API int mmj_colsum_bf16_static_max_n() { return kStaticColsumMaxN; }

MMJ_API const char* mmj_colsum_bf16_static_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case -1: return "mmj_colsum_bf16_static: leading dimension must be a multiple of 8 elements";
    case -20: return "mmj_colsum_bf16_static: N is larger than the built-in scratch allows (max 16384 columns)";
    case -21: return "mmj_colsum_bf16_static: device ordinal out of range";
    case -22: return "mmj_colsum_bf16_static: cudaGetSymbolAddress failed for the built-in scratch";
    default: return code > 0 ? "mmj_colsum_bf16_static: CUDA launch error" : "mmj_colsum_bf16_static: unknown error";
  }
}

MMJ_API int mmj_colsum_bf16_static(const void* x, long long ldx, void* out_bf16, float* out_f32,
                                   int M, int N, int accumulate, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (ldx % 8) return -1;
  if (N > kStaticColsumMaxN) return -20;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kStaticMaxDevices) return -21;
  float* scratch = g_colsum_static_ptr[dev];
  if (scratch == nullptr) {
    // one-time set-up for this device: translate the symbol into a device address
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_colsum_static_scratch);
    if (e != cudaSuccess || p == nullptr) return -22;
    scratch = static_cast<float*>(p);
    g_colsum_static_ptr[dev] = scratch;
  }
  const int S = mmj_colsum_splits(M);  // <= kStaticColsumMaxSplits
  dim3 grid((N + 63) / 64, S);
  colsum_partial_kernel<<<grid, 256, 0, STREAM>>>((const __nv_bfloat16*)x, ldx, scratch, M, N);
  colsum_finalize_kernel<<<(N + 31) / 32, dim3(32, 8), 0, STREAM>>>(scratch, (__nv_bfloat16*)out_bf16,
                                                              out_f32, S, N, accumulate);
  return (int)cudaGetLastError();
}

MMJ_API int mmj_cast_f32_to_bf16_2d(const float* src, long long lds, void* dst, long long ldd,
                                    long long rows, int cols, void* stream) {
  if (cols % 4 || lds % 4 || ldd % 4) return -1;
  if (rows == 0 || cols == 0) return 0;
  launch_pdl(cast_f32_to_bf16_2d_kernel, dim3(grid_for(rows * (cols / 4), 256)), dim3(256), 0, STREAM, src, lds,
             (__nv_bfloat16*)dst, ldd, rows, cols);
  return (int)cudaGetLastError();
}

MMJ_BOUNDS_READER(mmj_debug_bounds_elementwise)
