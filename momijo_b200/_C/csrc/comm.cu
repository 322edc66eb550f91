// Collectives written directly over NVLink peer memory (no NCCL inside): every rank holds a
// table of peer base pointers into a symmetric heap and a pad of int32 signal slots.
//
//   * barrier / signal primitives with bounded waits (status word on timeout, never a trap)
//   * F1  gradient reduce-scatter + 1/world scaling + AdamW on the local fp32 shard + bf16
//         parameter write-back, in ONE kernel (peer loads, or NVLS multimem.ld_reduce)
//   * parameter all-gather by peer pulls (ranges not covered by the GEMM-fused all-gather)
//   * two-shot all-reduce (reduce-scatter then all-gather through peer memory) for DDP buckets
//   * slot reduction that finishes the GEMM -> reduce-scatter epilogue
//   * MoE dispatch (router permute + all-to-all by peer stores) and combine (peer pulls +
//     weighted un-permute)
//
// These give real semantics to the reference's identity-valued facade
// (legacy/src/momijo/learn/distributed/collective.mojo:163-232) and to the ZeroStage1 stubs
// (legacy/src/momijo/learn/distributed/sharding.mojo:130-168).
//
// Signal protocol: slot values are monotonically increasing epochs. A producer publishes data
// with st.release.sys of the epoch; a consumer spins with ld.acquire.sys until the slot is
// >= the epoch it expects, for at most MMJ_WAIT_BUDGET_NS.
#include "common.cuh"

namespace mmj {

constexpr int kMaxWorld = 8;

__device__ __forceinline__ int ld_acq_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_rel_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait for *flag >= want (system scope). false on timeout.
__device__ __forceinline__ bool wait_sys_ge(const int* flag, int want, int* status, int detail) {
  if (ld_acq_sys(flag) >= want) return true;
  uint64_t t0 = 0;  // %globaltimer is slow to read: start the clock only after many polls
  uint32_t it = 0;
  while (true) {
    if (ld_acq_sys(flag) >= want) return true;
    __nanosleep(64);
    if (((++it) & 0xff) == 0) {
      if (status_failed(status)) return false;
      if (t0 == 0) {
        t0 = globaltimer_ns();
      } else if (globaltimer_ns() - t0 > MMJ_WAIT_BUDGET_NS) {
        report(status, kTimeoutBarrier, detail);
        return false;
      }
    }
  }
}

struct PeerTable {
  int world, rank;
  int* sig[kMaxWorld];  // signal pads of every rank (sig[rank] is local)
};

// Every rank writes `epoch` into slot (base + rank) of every peer, then waits until its own
// slots (base + r) hold >= epoch for all r. Called by ONE thread block; thread r < world signals.
__device__ __forceinline__ bool block_barrier(const PeerTable& t, int slot_base, int epoch,
                                              int* status, int* smem_ok) {
  if (threadIdx.x == 0) *smem_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < t.world) {
    __threadfence_system();
    st_rel_sys(t.sig[threadIdx.x] + slot_base + t.rank, epoch);
    if (!wait_sys_ge(t.sig[t.rank] + slot_base + threadIdx.x, epoch, status, threadIdx.x))
      *smem_ok = 0;
  }
  __syncthreads();
  return *smem_ok != 0;
}

__global__ void barrier_kernel(PeerTable t, int slot_base, int epoch, int* status) {
  __shared__ int ok;
  block_barrier(t, slot_base, epoch, status, &ok);
}

__global__ void signal_kernel(PeerTable t, int slot, int epoch) {
  if ((int)threadIdx.x < t.world) {
    __threadfence_system();
    st_rel_sys(t.sig[threadIdx.x] + slot, epoch);
  }
}

// Waits (bounded) for local slot >= epoch; used by tests of the timeout path and by consumers
// that need a stream-ordered wait on a peer's signal.
__global__ void wait_kernel(const int* slot, int epoch, int* status) {
  if (threadIdx.x == 0) wait_sys_ge(slot, epoch, status, -1);
}

// ---- helpers -----------------------------------------------------------------------------------
__device__ __forceinline__ void bf16x8_to_f32(const uint4& q, float (&f)[8]) {
  float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z),
         d = unpack_bf16x2(q.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 f32_to_bf16x8(const float (&f)[8]) {
  uint4 q;
  q.x = pack_bf16x2(f[0], f[1]);
  q.y = pack_bf16x2(f[2], f[3]);
  q.z = pack_bf16x2(f[4], f[5]);
  q.w = pack_bf16x2(f[6], f[7]);
  return q;
}
// In-switch reduction of 8 bf16 across all ranks bound to the multicast address (fp32 adds).
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 q;
  asm volatile(
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
      : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
      : "l"(mc_addr)
      : "memory");
  return q;
}

// Grid-wide "last block" detection with a wrapping counter.
__device__ __forceinline__ bool last_block_done(unsigned int* counter) {
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int old = atomicInc(counter, gridDim.x - 1);
    is_last = (old == gridDim.x - 1);
  }
  __syncthreads();
  return is_last != 0;
}

// ================================================================================================
// F1: reduce-scatter + scale + AdamW + bf16 write-back
// ================================================================================================
struct RsAdamwParams {
  PeerTable t;
  const __nv_bfloat16* grad[kMaxWorld];  // flat gradient buffer of every rank (peer pointers)
  const __nv_bfloat16* grad_mc;          // multicast address of the gradient buffer, or null
  __nv_bfloat16* param;                  // local flat parameter buffer
  float* master;                         // local shard, fp32
  float* m;
  float* v;
  long long shard_off;    // first element of the local shard in the flat buffers
  long long shard_elems;  // multiple of 8
  float lr, b1, b2, eps, wd, inv_bc1, inv_bc2, grad_scale;
  const float* grad_scale_dev;  // optional device factor on top of grad_scale (gradient clipping)
  float* reduced_out;     // optional [shard_elems] fp32: write the reduced, scaled gradient shard here
                          // and leave master / m / v / param untouched (the update then runs later,
                          // once a global gradient norm is known)
  int slot_base;          // uses slots [slot_base, slot_base + 2*world)
  int epoch;
  unsigned int* block_counter;
  float* sqnorm_out;  // optional: sum of squares of the reduced, scaled local gradient shard
  int* status;
};

__global__ void __launch_bounds__(256) rs_adamw_kernel(const RsAdamwParams p) {
  __shared__ int ok;
  // entry: every rank has finished writing its gradients. A block whose barrier ran out of time skips
  // the work but still takes part in the block count below, so the wrapping counter ends at zero.
  const bool entered = block_barrier(p.t, p.slot_base, p.epoch, p.status, &ok);

  const int W = p.t.world;
  float scale = p.grad_scale / (float)W;
  if (p.grad_scale_dev != nullptr) scale *= *p.grad_scale_dev;
  const long long nvec = entered ? (p.shard_elems >> 3) : 0;
  float sq = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long e = p.shard_off + i * 8;
    float acc[8];
    if (p.grad_mc != nullptr) {
      uint4 q = multimem_ld_reduce_bf16x8(p.grad_mc + e);
      bf16x8_to_f32(q, acc);
    } else {
      uint4 q[kMaxWorld];
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r)
        if (r < W) q[r] = *reinterpret_cast<const uint4*>(p.grad[(p.t.rank + r) % W] + e);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r)
        if (r < W) {
          float f[8];
          bf16x8_to_f32(q[r], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += f[j];
        }
    }
    if (p.reduced_out != nullptr) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc[j] *= scale;
        sq += acc[j] * acc[j];
      }
      *reinterpret_cast<float4*>(p.reduced_out + i * 8) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(p.reduced_out + i * 8 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
      continue;
    }
    float4 w0 = *reinterpret_cast<float4*>(p.master + i * 8), w1 = *reinterpret_cast<float4*>(p.master + i * 8 + 4);
    float4 m0 = *reinterpret_cast<float4*>(p.m + i * 8), m1 = *reinterpret_cast<float4*>(p.m + i * 8 + 4);
    float4 v0 = *reinterpret_cast<float4*>(p.v + i * 8), v1 = *reinterpret_cast<float4*>(p.v + i * 8 + 4);
    float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float g = acc[j] * scale;
      sq += g * g;
      mm[j] = p.b1 * mm[j] + (1.f - p.b1) * g;
      vv[j] = p.b2 * vv[j] + (1.f - p.b2) * g * g;
      const float upd = (mm[j] * p.inv_bc1) / (sqrtf(vv[j] * p.inv_bc2) + p.eps);
      w[j] = w[j] - p.lr * (upd + p.wd * w[j]);
    }
    *reinterpret_cast<float4*>(p.master + i * 8) = make_float4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<float4*>(p.master + i * 8 + 4) = make_float4(w[4], w[5], w[6], w[7]);
    *reinterpret_cast<float4*>(p.m + i * 8) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(p.m + i * 8 + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
    *reinterpret_cast<float4*>(p.v + i * 8) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    *reinterpret_cast<float4*>(p.v + i * 8 + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
    *reinterpret_cast<uint4*>(p.param + e) = f32_to_bf16x8(w);
  }
  if (p.sqnorm_out != nullptr) {
    sq = warp_sum(sq);
    if ((threadIdx.x & 31) == 0) atomicAdd(p.sqnorm_out, sq);
  }
  // exit: nobody leaves before every rank has finished pulling gradients and publishing its
  // parameter shard (so the next step may overwrite gradients and read peer parameters)
  if (last_block_done(p.block_counter) && entered)
    block_barrier(p.t, p.slot_base + W, p.epoch, p.status, &ok);
}

// ================================================================================================
// Bucket all-gather: a bucket of `world * shard_bytes` bytes is cut into one contiguous shard per
// rank. Each rank pulls the shards it does not own into dst (bucket layout: shard r at r * shard_bytes)
// from src[r] + r * src_stride (src_stride = shard_bytes when the peers keep the bucket in the same
// full layout, 0 when every peer keeps only its own shard in a compact buffer; copy_self then also
// copies the local shard). Up to four byte ranges of the bucket can be left out: the GEMM that
// consumes such a range first gathers it itself.
// ================================================================================================
struct GatherBucketParams {
  PeerTable t;
  const uint8_t* src[kMaxWorld];
  uint8_t* dst;
  long long shard_bytes, src_stride;
  long long skip_lo[4], skip_hi[4];
  int n_skip, copy_self;
  int slot_base, epoch;  // entry barrier slots (skipped when epoch < 0)
  int* status;
};

__global__ void __launch_bounds__(256) gather_bucket_kernel(const GatherBucketParams p) {
  __shared__ int ok;
  if (p.epoch >= 0 && !block_barrier(p.t, p.slot_base, p.epoch, p.status, &ok)) return;
  const long long n16 = p.shard_bytes >> 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (int rr = 0; rr < p.t.world; ++rr) {
    const int r = (p.t.rank + rr) % p.t.world;  // every rank starts at a different owner
    if (r == p.t.rank && !p.copy_self) continue;
    const uint8_t* s = p.src[r] + (long long)r * p.src_stride;
    uint8_t* d = p.dst + (long long)r * p.shard_bytes;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n16; i += stride) {
      const long long off = (long long)r * p.shard_bytes + (i << 4);
      bool skip = false;
      for (int k = 0; k < p.n_skip; ++k) skip |= (off >= p.skip_lo[k] && off < p.skip_hi[k]);
      if (skip) continue;
      *reinterpret_cast<uint4*>(d + (i << 4)) = *reinterpret_cast<const uint4*>(s + (i << 4));
    }
  }
}

// ================================================================================================
// Small fp32 all-reduce (sum) of n <= 64 values: every rank stores its values into slot `rank` of
// every peer's staging buffer ([world][64] floats, symmetric), one barrier, then each rank adds the
// world slots in rank order (the same order everywhere: bitwise equal results on every rank). Single
// block. Used for gradient-norm and loss-statistic scalars, where a library collective's launch and
// synchronisation would cost more than the data.
// ================================================================================================
struct SmallAllReduceParams {
  PeerTable t;
  float* stage[kMaxWorld];
  const float* in;
  float* out;
  int n;
  int slot_base, epoch;
  int* status;
};

__global__ void __launch_bounds__(64) allreduce_small_kernel(const SmallAllReduceParams p) {
  __shared__ int ok;
  const int W = p.t.world;
  // two staging halves used alternately: a rank may start the next call while a slow peer still
  // reads the values of this one
  const int half = (p.epoch & 1) * kMaxWorld * 64;
  if ((int)threadIdx.x < p.n) {
    const float v = p.in[threadIdx.x];
    for (int r = 0; r < W; ++r) p.stage[r][half + p.t.rank * 64 + threadIdx.x] = v;
  }
  __threadfence_system();
  if (!block_barrier(p.t, p.slot_base, p.epoch, p.status, &ok)) return;
  if ((int)threadIdx.x < p.n) {
    float s = 0.f;
    const volatile float* mine = p.stage[p.t.rank] + half;
    for (int r = 0; r < W; ++r) s += mine[r * 64 + threadIdx.x];
    p.out[threadIdx.x] = s;
  }
}

// ================================================================================================
// Parameter all-gather by pulls: for every byte range [lo, hi) of the flat buffer, copy the
// pieces owned by other ranks (owner = offset / shard_bytes) from the owner's buffer.
// ================================================================================================
struct AllGatherParams {
  PeerTable t;
  const uint8_t* src[kMaxWorld];
  uint8_t* dst;
  long long shard_bytes;
  const long long* ranges;  // [n_ranges][2] byte offsets, 16-byte aligned
  int n_ranges;
  int slot_base, epoch;     // entry barrier slots (skipped when epoch < 0)
  int* status;
};

__global__ void __launch_bounds__(256) allgather_ranges_kernel(const AllGatherParams p) {
  __shared__ int ok;
  if (p.epoch >= 0 && !block_barrier(p.t, p.slot_base, p.epoch, p.status, &ok)) return;
  for (int ri = 0; ri < p.n_ranges; ++ri) {
    const long long lo = p.ranges[2 * ri], hi = p.ranges[2 * ri + 1];
    const long long n16 = (hi - lo) >> 4;
    long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    // four independent 16-byte loads per thread and trip: one NVLink round trip (2-3 us) per trip,
    // so a thread that waits for each load before asking for the next leaves the links mostly idle
    for (; i + 3 * stride < n16; i += 4 * stride) {
      uint4 q[4];
      long long off[4];
      bool mine[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        off[u] = lo + ((i + u * stride) << 4);
        const int owner = (int)(off[u] / p.shard_bytes);
        mine[u] = owner == p.t.rank;
        if (!mine[u]) q[u] = *reinterpret_cast<const uint4*>(p.src[owner] + off[u]);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (!mine[u]) *reinterpret_cast<uint4*>(p.dst + off[u]) = q[u];
    }
    for (; i < n16; i += stride) {
      const long long off = lo + (i << 4);
      const int owner = (int)(off / p.shard_bytes);
      if (owner == p.t.rank) continue;
      *reinterpret_cast<uint4*>(p.dst + off) = *reinterpret_cast<const uint4*>(p.src[owner] + off);
    }
  }
}

// ================================================================================================
// Two-shot all-reduce on a symmetric bf16 buffer (sum, optional scale): phase 1 each rank
// reduces its slice from all peers into its own buffer; cross-GPU barrier; phase 2 each rank
// pulls the other slices. One kernel; grid must be resident (<= SM count x occupancy).
// ================================================================================================
struct AllReduceParams {
  PeerTable t;
  __nv_bfloat16* buf[kMaxWorld];
  const __nv_bfloat16* buf_mc;
  long long n;  // elements, multiple of 8 * world
  float scale;
  int slot_base, epoch;
  unsigned int* block_counter;  // two counters
  int* grid_flag;               // local int: set to epoch when the mid barrier has completed
  int* status;
};

__global__ void __launch_bounds__(256) allreduce_kernel(const AllReduceParams p) {
  __shared__ int ok;
  if (!block_barrier(p.t, p.slot_base, p.epoch, p.status, &ok)) return;
  const int W = p.t.world, R = p.t.rank;
  const long long slice = p.n / W;
  const long long nvec = slice >> 3;
  __nv_bfloat16* mine = p.buf[R] + (long long)R * slice;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[8];
    if (p.buf_mc != nullptr) {
      uint4 q = multimem_ld_reduce_bf16x8(p.buf_mc + (long long)R * slice + i * 8);
      bf16x8_to_f32(q, acc);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int r = 0; r < W; ++r) {
        uint4 q = *reinterpret_cast<const uint4*>(p.buf[(R + r) % W] + (long long)R * slice + i * 8);
        float f[8];
        bf16x8_to_f32(q, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= p.scale;
    *reinterpret_cast<uint4*>(mine + i * 8) = f32_to_bf16x8(acc);
  }
  // mid barrier: the last block to finish phase 1 runs the cross-GPU barrier and releases the
  // others through a local flag
  if (last_block_done(p.block_counter)) {
    const bool good = block_barrier(p.t, p.slot_base + W, p.epoch, p.status, &ok);
    if (threadIdx.x == 0) {
      __threadfence();
      atomicExch(p.grid_flag, good ? p.epoch : -p.epoch);
    }
  }
  __shared__ int go;
  if (threadIdx.x == 0) {
    go = 1;
    const uint64_t t0 = globaltimer_ns();
    while (true) {
      int v = *reinterpret_cast<volatile int*>(p.grid_flag);
      if (v == p.epoch) break;
      if (v == -p.epoch) { go = 0; break; }
      __nanosleep(100);
      if (globaltimer_ns() - t0 > MMJ_WAIT_BUDGET_NS) {
        report(p.status, kTimeoutBarrier, 77);
        go = 0;
        break;
      }
    }
    __threadfence();
  }
  __syncthreads();
  if (!go) return;
  for (int r = 1; r < W; ++r) {
    const int src = (R + r) % W;
    const uint4* s = reinterpret_cast<const uint4*>(p.buf[src] + (long long)src * slice);
    uint4* d = reinterpret_cast<uint4*>(p.buf[R] + (long long)src * slice);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x)
      d[i] = s[i];
  }
  // exit barrier: peers may overwrite their buffers only after everyone has pulled
  if (last_block_done(p.block_counter + 1))
    block_barrier(p.t, p.slot_base + 2 * W, p.epoch, p.status, &ok);
}

// ================================================================================================
// Slot reduction for GEMM -> reduce-scatter: out[r, c] = sum_s stage[s][r, c]
// ================================================================================================
__global__ void __launch_bounds__(256)
reduce_slots_kernel(PeerTable t, const __nv_bfloat16* stage, long long slot_stride,
                    __nv_bfloat16* out, const __nv_bfloat16* residual, long long n, int slot_base,
                    int epoch, int* status) {
  __shared__ int ok;
  // all peers have finished their GEMM epilogues (stores into this rank's slots)
  if (!block_barrier(t, slot_base, epoch, status, &ok)) return;
  const long long nvec = n >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < t.world; ++s) {
      float f[8];
      bf16x8_to_f32(*reinterpret_cast<const uint4*>(stage + s * slot_stride + i * 8), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    if (residual != nullptr) {
      float f[8];
      bf16x8_to_f32(*reinterpret_cast<const uint4*>(residual + i * 8), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    *reinterpret_cast<uint4*>(out + i * 8) = f32_to_bf16x8(acc);
  }
}

// ================================================================================================
// Reduce-scatter by pulls: every rank holds a full partial product [world * n] in symmetric memory
// and sums its own block of n elements over all ranks (peer loads), plus an optional residual.
// The unfused counterpart of GEMM -> reduce-scatter for products of a few thousand rows, where the
// epilogue's 64-byte peer stores and the slot pass cost more than a plain GEMM followed by this.
// ================================================================================================
struct ReducePullParams {
  PeerTable t;
  const __nv_bfloat16* src[kMaxWorld];  // every rank's partial buffer
  __nv_bfloat16* out;                   // [n]
  const __nv_bfloat16* residual;        // [n] or null
  long long n;                          // elements of one block, multiple of 8
  int slot_base, epoch;
  int* status;
};

__global__ void __launch_bounds__(256) reduce_pull_kernel(const ReducePullParams p) {
  __shared__ int ok;
  // every rank's product is complete (its GEMM precedes this kernel in stream order)
  if (!block_barrier(p.t, p.slot_base, p.epoch, p.status, &ok)) return;
  const int W = p.t.world;
  const long long nvec = p.n >> 3;
  const long long base = (long long)p.t.rank * p.n;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    // all loads of a vector are requested before the first is used; ranks are added in the order
    // 0..W-1 on every rank, so the sum does not depend on who owns the block
    uint4 q[kMaxWorld];
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
      if (r < W) q[r] = *reinterpret_cast<const uint4*>(p.src[r] + base + i * 8);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (p.residual != nullptr) bf16x8_to_f32(*reinterpret_cast<const uint4*>(p.residual + i * 8), acc);
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r) {
      if (r < W) {
        float f[8];
        bf16x8_to_f32(q[r], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
    }
    *reinterpret_cast<uint4*>(p.out + i * 8) = f32_to_bf16x8(acc);
  }
}

// ================================================================================================
// MoE dispatch / combine
// ================================================================================================
// Layout on every rank (symmetric): recv buffer [cap_rows, H] bf16 holding, for each local
// expert, one segment per source rank; segment starts come from the exchanged count table.
//
// Step 1 (count): each rank histograms its (token, k) assignments per global expert and writes
//   counts[src_rank][expert] into every peer's count table (peer stores), then barrier.
// Step 2 (offsets, local): for local expert e and source s, seg_off[e][s] = running sum padded so
//   that each expert starts on a 128-row boundary; also tile_group[] and num_m_tiles for the
//   grouped GEMM. Every rank computes the offsets of ALL ranks (the table is replicated), so a
//   sender knows where its rows go without another exchange.
// Step 3 (dispatch): each (token, k) row is written straight into the destination rank's recv
//   buffer at seg_off + position (peer stores), then barrier.
// Combine: out[token] = sum_k w[token,k] * expert_out[dest_rank][row]  (peer pulls).

struct MoeCountParams {
  PeerTable t;
  const int* expert_idx;  // [n_assign] global expert of each (token, k)
  int n_assign;
  int n_experts;           // global
  int* counts[kMaxWorld];  // counts[r]: rank r's table [world][n_experts] (peer pointers)
  int* local_pos;          // [n_assign] position of the assignment inside its (src, expert) run
  int slot_base, epoch;
  int* status;
};

// Single-block histogram (n_assign is a few 100k at most; shared-memory atomics).
__global__ void __launch_bounds__(1024) moe_count_kernel(const MoeCountParams p) {
  extern __shared__ int hist[];  // n_experts
  __shared__ int ok;
  for (int e = threadIdx.x; e < p.n_experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < p.n_assign; i += blockDim.x) {
    const int e = p.expert_idx[i];
    if (!index_ok(e, p.n_experts, /*site=*/10)) {   // a router index outside [0, E): counted nowhere
      p.local_pos[i] = 0;
      continue;
    }
    p.local_pos[i] = atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < p.n_experts; e += blockDim.x) {
    const int c = hist[e];
    for (int r = 0; r < p.t.world; ++r) p.counts[r][p.t.rank * p.n_experts + e] = c;
  }
  __syncthreads();
  block_barrier(p.t, p.slot_base, p.epoch, p.status, &ok);
}

// offsets for every (dest rank, local expert, src rank); one block.
// seg_off: [world(dest)][experts_per_rank][world(src)] row offsets inside dest's recv buffer
// tile_group / num_tiles describe THIS rank's recv buffer for the grouped GEMM.
__global__ void moe_offsets_kernel(const int* counts, int world, int rank, int n_experts,
                                   int* seg_off, int* tile_group, int* num_tiles, int* total_rows,
                                   int* pad_ranges, int* expert_ranges, int max_tiles) {
  if (threadIdx.x != 0) return;
  const int epr = n_experts / world;
  for (int d = 0; d < world; ++d) {
    int row = 0;
    for (int le = 0; le < epr; ++le) {
      const int e = d * epr + le;
      const int start = row;
      for (int s = 0; s < world; ++s) {
        seg_off[(d * epr + le) * world + s] = row;
        row += counts[s * n_experts + e];
      }
      const int padded = (row + 127) / 128 * 128;
      if (d == rank) {
        for (int tI = start / 128; tI < padded / 128 && tI < max_tiles; ++tI) tile_group[tI] = le;
        const int cap = max_tiles * 128;   // rows past the buffer's capacity are dropped
        pad_ranges[2 * le] = min(row, cap);          // rows [row, padded) of this expert hold no token
        pad_ranges[2 * le + 1] = min(padded, cap);
        expert_ranges[2 * le] = min(start, cap);     // rows [start, padded) belong to this expert
        expert_ranges[2 * le + 1] = min(padded, cap);
      }
      row = padded;
    }
    if (d == rank) {
      *num_tiles = min(row / 128, max_tiles);
      *total_rows = min(row, max_tiles * 128);
    }
  }
}

__global__ void moe_zero_pad_kernel(__nv_bfloat16* buf, int H, const int* pad_ranges, int cap_rows) {
  const int lo = pad_ranges[2 * blockIdx.x], hi = min(pad_ranges[2 * blockIdx.x + 1], cap_rows);
  const long long n16 = (long long)max(hi - lo, 0) * H / 8;
  uint4* p = reinterpret_cast<uint4*>(buf + (long long)lo * H);
  for (long long i = threadIdx.x; i < n16; i += blockDim.x) p[i] = make_uint4(0, 0, 0, 0);
}

// dgate[a] = <dout[token(a)], y[row(a)]>  (gradient of the router weight of assignment a)
struct MoeGateGradParams {
  const __nv_bfloat16* y[kMaxWorld];
  const __nv_bfloat16* dout;
  const int* expert_idx;
  const int* src_row_of;
  float* dgate;
  int n_assign, top_k, H, epr;
};
__global__ void __launch_bounds__(256) moe_gate_grad_kernel(const MoeGateGradParams p) {
  const int lane = threadIdx.x & 31;
  const int a = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (a >= p.n_assign) return;
  const int d = p.expert_idx[a] / p.epr;
  if (p.src_row_of[a] < 0) {  // dropped at capacity
    if (lane == 0) p.dgate[a] = 0.f;
    return;
  }
  const uint4* yr = reinterpret_cast<const uint4*>(p.y[d] + (long long)p.src_row_of[a] * p.H);
  const uint4* gr = reinterpret_cast<const uint4*>(p.dout + (long long)(a / p.top_k) * p.H);
  float s = 0.f;
  for (int c = lane; c < (p.H >> 3); c += 32) {
    float f[8], g[8];
    bf16x8_to_f32(yr[c], f);
    bf16x8_to_f32(gr[c], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += f[j] * g[j];
  }
  s = warp_sum(s);
  if (lane == 0) p.dgate[a] = s;
}

struct MoeDispatchParams {
  PeerTable t;
  const __nv_bfloat16* x;  // [n_tokens, H]
  const int* expert_idx;   // [n_assign]
  const int* local_pos;    // [n_assign]
  const int* seg_off;      // [world][epr][world]
  __nv_bfloat16* recv[kMaxWorld];  // recv buffers of all ranks
  int* src_row_of;         // [n_assign] out: row index inside the destination's recv buffer
  const float* row_w;      // optional [n_assign]: rows are scaled on the way out
  int cap_rows;            // rows available in every recv buffer
  int n_assign, top_k, H, n_experts;
  int slot_base, epoch;
  unsigned int* block_counter;
  int* status;
};

__global__ void __launch_bounds__(256) moe_dispatch_kernel(const MoeDispatchParams p) {
  __shared__ int ok;
  const int W = p.t.world, epr = p.n_experts / W;
  const int h8 = p.H >> 3;
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int a = blockIdx.x * warps_per_block + (threadIdx.x >> 5); a < p.n_assign;
       a += gridDim.x * warps_per_block) {
    const int e = p.expert_idx[a];
    if (!index_ok(e, p.n_experts, /*site=*/11)) {
      if (lane == 0) p.src_row_of[a] = -1;
      continue;
    }
    const int d = e / epr, le = e - d * epr;
    const int row = p.seg_off[(d * epr + le) * W + p.t.rank] + p.local_pos[a];
    if (row >= p.cap_rows || row < 0) {  // over capacity: the assignment is dropped (contributes nothing)
      if (lane == 0) p.src_row_of[a] = -1;
      continue;
    }
    if (lane == 0) p.src_row_of[a] = row;
    const uint4* s = reinterpret_cast<const uint4*>(p.x + (long long)(a / p.top_k) * p.H);
    uint4* dst = reinterpret_cast<uint4*>(p.recv[d] + (long long)row * p.H);
    if (p.row_w == nullptr) {
      for (int c = lane; c < h8; c += 32) dst[c] = s[c];
    } else {
      const float w = p.row_w[a];
      for (int c = lane; c < h8; c += 32) {
        float f[8];
        bf16x8_to_f32(s[c], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] *= w;
        dst[c] = f32_to_bf16x8(f);
      }
    }
  }
  if (last_block_done(p.block_counter)) block_barrier(p.t, p.slot_base, p.epoch, p.status, &ok);
}

struct MoeCombineParams {
  PeerTable t;
  const __nv_bfloat16* y[kMaxWorld];  // expert outputs (recv-buffer layout) of all ranks
  const int* expert_idx;
  const int* src_row_of;
  const float* gate_w;  // [n_assign] router weights
  __nv_bfloat16* out;   // [n_tokens, H]
  const __nv_bfloat16* residual;  // optional [n_tokens, H] (shared-expert output etc.)
  int n_tokens, top_k, H, n_experts;
  int cap_rows;          // rows of every rank's expert-output buffer (bound of src_row_of)
  int slot_base, epoch;  // entry barrier: all ranks' expert outputs are complete
  int* status;
};

__global__ void __launch_bounds__(256) moe_combine_kernel(const MoeCombineParams p) {
  __shared__ int ok;
  if (p.epoch >= 0 && !block_barrier(p.t, p.slot_base, p.epoch, p.status, &ok)) return;
  const int W = p.t.world, epr = p.n_experts / W;
  const int h8 = p.H >> 3;
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int tk = blockIdx.x * warps_per_block + (threadIdx.x >> 5); tk < p.n_tokens;
       tk += gridDim.x * warps_per_block) {
    for (int c = lane; c < h8; c += 32) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (p.residual != nullptr)
        bf16x8_to_f32(*reinterpret_cast<const uint4*>(p.residual + (long long)tk * p.H + c * 8), acc);
      for (int k = 0; k < p.top_k; ++k) {
        const int a = tk * p.top_k + k;
        if (!index_ok(p.expert_idx[a], p.n_experts, /*site=*/12)) continue;
        const int d = p.expert_idx[a] / epr;
        if (p.src_row_of[a] < 0) continue;  // dropped at capacity
        if (!index_ok(p.src_row_of[a], p.cap_rows, /*site=*/13)) continue;
        const float w = (p.gate_w != nullptr) ? p.gate_w[a] : 1.0f;
        float f[8];
        bf16x8_to_f32(*reinterpret_cast<const uint4*>(p.y[d] + (long long)p.src_row_of[a] * p.H + c * 8), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += w * f[j];
      }
      *reinterpret_cast<uint4*>(p.out + (long long)tk * p.H + c * 8) = f32_to_bf16x8(acc);
    }
  }
}

static PeerTable make_table(int world, int rank, void* const* sig) {
  PeerTable t;
  t.world = world;
  t.rank = rank;
  for (int r = 0; r < kMaxWorld; ++r) t.sig[r] = (r < world) ? (int*)sig[r] : nullptr;
  return t;
}

static int resident_grid(int per_sm) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms * per_sm;
}

// Signal pads have a fixed number of int32 slots (set once by the communicator). Every launcher checks the
// slot range a kernel is about to use on the host, before the launch: a range past the pad would make a
// peer store land in whatever follows the pad in the peer's heap.
static int g_signal_slots = 0;
static inline bool slots_ok(int slot_base, int count) {
  if (slot_base < 0 || count < 0) return false;
  return g_signal_slots == 0 || slot_base + count <= g_signal_slots;
}

}  // namespace mmj

using namespace mmj;
#define STREAM ((cudaStream_t)stream)

MMJ_API int mmj_set_signal_slots(int n) {
  g_signal_slots = n > 0 ? n : 0;
  return 0;
}

MMJ_BOUNDS_READER(mmj_debug_bounds_comm)

MMJ_API int mmj_barrier(void* const* sig, int world, int rank, int slot_base, int epoch,
                        int* status, void* stream) {
  if (world < 1 || world > kMaxWorld) return -1;
  if (!slots_ok(slot_base, world)) return -9;
  barrier_kernel<<<1, 32, 0, STREAM>>>(make_table(world, rank, sig), slot_base, epoch, status);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_signal_peers(void* const* sig, int world, int rank, int slot, int epoch,
                             void* stream) {
  if (world < 1 || world > kMaxWorld) return -1;
  signal_kernel<<<1, 32, 0, STREAM>>>(make_table(world, rank, sig), slot, epoch);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_wait_flag(const int* slot, int epoch, int* status, void* stream) {
  wait_kernel<<<1, 32, 0, STREAM>>>(slot, epoch, status);
  return (int)cudaGetLastError();
}

MMJ_API int mmj_rs_adamw(void* const* sig, void* const* grads, const void* grad_mc, void* param,
                         float* master, float* m, float* v, long long shard_off,
                         long long shard_elems, float lr, float b1, float b2, float eps, float wd,
                         float bc1, float bc2, float grad_scale, const float* grad_scale_dev,
                         float* reduced_out, int max_blocks, int world, int rank, int slot_base,
                         int epoch, unsigned int* block_counter, float* sqnorm_out, int* status,
                         void* stream) {
  if (world < 1 || world > kMaxWorld) return -1;
  if (!slots_ok(slot_base, 2 * world)) return -9;
  if (shard_elems % 8 || shard_off % 8) return -2;
  RsAdamwParams p;
  p.t = make_table(world, rank, sig);
  for (int r = 0; r < kMaxWorld; ++r) p.grad[r] = (r < world) ? (const __nv_bfloat16*)grads[r] : nullptr;
  p.grad_mc = (const __nv_bfloat16*)grad_mc;
  p.param = (__nv_bfloat16*)param;
  p.master = master; p.m = m; p.v = v;
  p.shard_off = shard_off; p.shard_elems = shard_elems;
  p.lr = lr; p.b1 = b1; p.b2 = b2; p.eps = eps; p.wd = wd;
  p.inv_bc1 = 1.0f / bc1; p.inv_bc2 = 1.0f / bc2;
  p.grad_scale = grad_scale;
  p.grad_scale_dev = grad_scale_dev;
  p.reduced_out = reduced_out;
  p.slot_base = slot_base; p.epoch = epoch;
  p.block_counter = block_counter;
  p.sqnorm_out = sqnorm_out;
  p.status = status;
  long long want = (shard_elems / 8 + 255) / 256;
  int grid = resident_grid(4);
  // a launch that runs beside the backward pass is given fewer blocks, so that it does not crowd
  // the GEMM CTAs out of issue slots and memory bandwidth
  if (max_blocks > 0 && max_blocks < grid) grid = max_blocks;
  if (want < grid) grid = (int)(want < 1 ? 1 : want);
  rs_adamw_kernel<<<grid, 256, 0, STREAM>>>(p);
  return (int)cudaGetLastError();
}

MMJ_API int mmj_gather_bucket(void* const* sig, void* const* srcs, void* dst, long long shard_bytes,
                              long long src_stride, const long long* skip_ranges, int n_skip,
                              int copy_self, int max_blocks, int world, int rank, int slot_base,
                              int epoch, int* status, void* stream) {
  if (world < 1 || world > kMaxWorld) return -1;
  if (epoch >= 0 && !slots_ok(slot_base, world)) return -9;
  if ((shard_bytes & 15) || (src_stride & 15) || n_skip < 0 || n_skip > 4) return -2;
  GatherBucketParams p;
  p.t = make_table(world, rank, sig);
  for (int r = 0; r < kMaxWorld; ++r) p.src[r] = (r < world) ? (const uint8_t*)srcs[r] : nullptr;
  p.dst = (uint8_t*)dst;
  p.shard_bytes = shard_bytes;
  p.src_stride = src_stride;
  for (int k = 0; k < 4; ++k) {
    p.skip_lo[k] = (k < n_skip) ? skip_ranges[2 * k] : 0;       // host array
    p.skip_hi[k] = (k < n_skip) ? skip_ranges[2 * k + 1] : 0;
  }
  p.n_skip = n_skip;
  p.copy_self = copy_self;
  p.slot_base = slot_base; p.epoch = epoch;
  p.status = status;
  int grid = resident_grid(2);
  if (max_blocks > 0 && max_blocks < grid) grid = max_blocks;
  long long want = (shard_bytes / 16 + 255) / 256;
  if (want < grid) grid = (int)(want < 1 ? 1 : want);
  gather_bucket_kernel<<<grid, 256, 0, STREAM>>>(p);
  return (int)cudaGetLastError();
}

// stage[r]: rank r's staging buffer of 2 * 8 * 64 floats (symmetric); in / out: n <= 64 local floats.
MMJ_API int mmj_allreduce_small_f32(void* const* sig, void* const* stage, const float* in, float* out,
                                    int n, int world, int rank, int slot_base, int epoch, int* status,
                                    void* stream) {
  if (world < 1 || world > kMaxWorld) return -1;
  if (!slots_ok(slot_base, world)) return -9;
  if (n < 1 || n > 64) return -2;
  SmallAllReduceParams p;
  p.t = make_table(world, rank, sig);
  for (int r = 0; r < kMaxWorld; ++r) p.stage[r] = (r < world) ? (float*)stage[r] : nullptr;
  p.in = in; p.out = out; p.n = n;
  p.slot_base = slot_base; p.epoch = epoch;
  p.status = status;
  allreduce_small_kernel<<<1, 64, 0, STREAM>>>(p);
  return (int)cudaGetLastError();
}

MMJ_API int mmj_allgather_ranges(void* const* sig, void* const* bufs, long long shard_bytes,
                                 const long long* ranges_dev, int n_ranges, int world, int rank,
                                 int slot_base, int epoch, int* status, void* stream) {
  if (world < 1 || world > kMaxWorld) return -1;
  if (epoch >= 0 && !slots_ok(slot_base, world)) return -9;
  AllGatherParams p;
  p.t = make_table(world, rank, sig);
  for (int r = 0; r < kMaxWorld; ++r) p.src[r] = (r < world) ? (const uint8_t*)bufs[r] : nullptr;
  p.dst = (uint8_t*)bufs[rank];
  p.shard_bytes = shard_bytes;
  p.ranges = ranges_dev;
  p.n_ranges = n_ranges;
  p.slot_base = slot_base; p.epoch = epoch;
  p.status = status;
  allgather_ranges_kernel<<<resident_grid(4), 256, 0, STREAM>>>(p);
  return (int)cudaGetLastError();
}

MMJ_API int mmj_allreduce_bf16(void* const* sig, void* const* bufs, const void* buf_mc, long long n,
                               float scale, int max_blocks, int world, int rank, int slot_base, int epoch,
                               unsigned int* block_counters, int* grid_flag, int* status,
                               void* stream) {
  if (world < 1 || world > kMaxWorld) return -1;
  if (!slots_ok(slot_base, 3 * world)) return -9;
  if (n % (8 * world)) return -2;
  AllReduceParams p;
  p.t = make_table(world, rank, sig);
  for (int r = 0; r < kMaxWorld; ++r) p.buf[r] = (r < world) ? (__nv_bfloat16*)bufs[r] : nullptr;
  p.buf_mc = (const __nv_bfloat16*)buf_mc;
  p.n = n; p.scale = scale;
  p.slot_base = slot_base; p.epoch = epoch;
  p.block_counter = block_counters;
  p.grid_flag = grid_flag;
  p.status = status;
  // every block spins on a flag set by another block: the whole grid must be resident
  int grid = resident_grid(2);
  // beside a running GEMM only part of that fits on the SMs at once: such launches ask for fewer blocks
  if (max_blocks > 0 && max_blocks < grid) grid = max_blocks;
  long long want = (n / world / 8 + 255) / 256;
  if (want < grid) grid = (int)(want < 1 ? 1 : want);
  allreduce_kernel<<<grid, 256, 0, STREAM>>>(p);
  return (int)cudaGetLastError();
}

MMJ_API int mmj_reduce_pull_bf16(void* const* sig, void* const* partials, void* out, const void* residual,
                                 long long n, int world, int rank, int slot_base, int epoch, int* status,
                                 void* stream) {
  if (world < 1 || world > kMaxWorld) return -1;
  if (!slots_ok(slot_base, world)) return -9;
  if (n % 8) return -2;
  ReducePullParams p;
  p.t = make_table(world, rank, sig);
  for (int r = 0; r < kMaxWorld; ++r) p.src[r] = (r < world) ? (const __nv_bfloat16*)partials[r] : nullptr;
  p.out = (__nv_bfloat16*)out;
  p.residual = (const __nv_bfloat16*)residual;
  p.n = n;
  p.slot_base = slot_base; p.epoch = epoch;
  p.status = status;
  long long want = (n / 8 + 255) / 256;
  int grid = resident_grid(4);
  if (want < grid) grid = (int)(want < 1 ? 1 : want);
  reduce_pull_kernel<<<grid, 256, 0, STREAM>>>(p);
  return (int)cudaGetLastError();
}

MMJ_API int mmj_reduce_slots_bf16(void* const* sig, const void* stage, long long slot_stride,
                                  void* out, const void* residual, long long n, int world, int rank,
                                  int slot_base, int epoch, int* status, void* stream) {
  if (world < 1 || world > kMaxWorld) return -1;
  if (!slots_ok(slot_base, world)) return -9;
  if (n % 8 || slot_stride % 8) return -2;
  long long want = (n / 8 + 255) / 256;
  int grid = resident_grid(4);
  if (want < grid) grid = (int)(want < 1 ? 1 : want);
  reduce_slots_kernel<<<grid, 256, 0, STREAM>>>(make_table(world, rank, sig),
                                                (const __nv_bfloat16*)stage, slot_stride,
                                                (__nv_bfloat16*)out, (const __nv_bfloat16*)residual,
                                                n, slot_base, epoch, status);
  return (int)cudaGetLastError();
}

MMJ_API int mmj_moe_count(void* const* sig, const int* expert_idx, int n_assign, int n_experts,
                          void* const* counts, int* local_pos, int world, int rank, int slot_base,
                          int epoch, int* status, void* stream) {
  if (world < 1 || world > kMaxWorld) return -1;
  if (!slots_ok(slot_base, world)) return -9;
  MoeCountParams p;
  p.t = make_table(world, rank, sig);
  p.expert_idx = expert_idx;
  p.n_assign = n_assign;
  p.n_experts = n_experts;
  for (int r = 0; r < kMaxWorld; ++r) p.counts[r] = (r < world) ? (int*)counts[r] : nullptr;
  p.local_pos = local_pos;
  p.slot_base = slot_base; p.epoch = epoch;
  p.status = status;
  moe_count_kernel<<<1, 1024, n_experts * sizeof(int), STREAM>>>(p);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_moe_offsets(const int* counts, int world, int rank, int n_experts, int* seg_off,
                            int* tile_group, int* num_tiles, int* total_rows, int* pad_ranges,
                            int* expert_ranges, int max_tiles, void* stream) {
  moe_offsets_kernel<<<1, 32, 0, STREAM>>>(counts, world, rank, n_experts, seg_off, tile_group,
                                           num_tiles, total_rows, pad_ranges, expert_ranges,
                                           max_tiles);
  return (int)cudaGetLastError();
}
// Zero the padding rows of a recv-layout buffer (rows that no token maps to), so that they add
// nothing when the rows are a contraction dimension (expert weight gradients).
MMJ_API int mmj_moe_zero_pad(void* buf, int H, const int* pad_ranges, int n_local_experts,
                             int cap_rows, void* stream) {
  moe_zero_pad_kernel<<<n_local_experts, 256, 0, STREAM>>>((__nv_bfloat16*)buf, H, pad_ranges,
                                                          cap_rows);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_moe_gate_grad(void* const* y, const void* dout, const int* expert_idx,
                              const int* src_row_of, float* dgate, int n_assign, int top_k, int H,
                              int n_experts, int world, void* stream) {
  if (world < 1 || world > kMaxWorld) return -1;
  MoeGateGradParams p;
  for (int r = 0; r < kMaxWorld; ++r) p.y[r] = (r < world) ? (const __nv_bfloat16*)y[r] : nullptr;
  p.dout = (const __nv_bfloat16*)dout;
  p.expert_idx = expert_idx; p.src_row_of = src_row_of; p.dgate = dgate;
  p.n_assign = n_assign; p.top_k = top_k; p.H = H; p.epr = n_experts / world;
  int grid = (n_assign + 7) / 8;
  if (grid < 1) grid = 1;
  moe_gate_grad_kernel<<<grid, 256, 0, STREAM>>>(p);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_moe_dispatch(void* const* sig, const void* x, const int* expert_idx,
                             const int* local_pos, const int* seg_off, void* const* recv,
                             int* src_row_of, const float* row_w, int cap_rows, int n_assign,
                             int top_k, int H, int n_experts,
                             int world, int rank, int slot_base, int epoch,
                             unsigned int* block_counter, int* status, void* stream) {
  if (world < 1 || world > kMaxWorld) return -1;
  if (!slots_ok(slot_base, world)) return -9;
  if (H % 8) return -2;
  MoeDispatchParams p;
  p.t = make_table(world, rank, sig);
  p.x = (const __nv_bfloat16*)x;
  p.expert_idx = expert_idx; p.local_pos = local_pos; p.seg_off = seg_off;
  for (int r = 0; r < kMaxWorld; ++r) p.recv[r] = (r < world) ? (__nv_bfloat16*)recv[r] : nullptr;
  p.src_row_of = src_row_of;
  p.row_w = row_w;
  p.cap_rows = cap_rows;
  p.n_assign = n_assign; p.top_k = top_k; p.H = H; p.n_experts = n_experts;
  p.slot_base = slot_base; p.epoch = epoch;
  p.block_counter = block_counter;
  p.status = status;
  int grid = resident_grid(4);
  int want = (n_assign + 7) / 8;
  if (want < grid) grid = want < 1 ? 1 : want;
  moe_dispatch_kernel<<<grid, 256, 0, STREAM>>>(p);
  return (int)cudaGetLastError();
}
MMJ_API int mmj_moe_combine(void* const* sig, void* const* y, const int* expert_idx,
                            const int* src_row_of, const float* gate_w, void* out,
                            const void* residual, int n_tokens, int top_k, int H, int n_experts,
                            int cap_rows, int world, int rank, int slot_base, int epoch, int* status,
                            void* stream) {
  if (world < 1 || world > kMaxWorld) return -1;
  if (H % 8) return -2;
  if (epoch >= 0 && !slots_ok(slot_base, world)) return -9;
  MoeCombineParams p;
  p.t = make_table(world, rank, sig);
  for (int r = 0; r < kMaxWorld; ++r) p.y[r] = (r < world) ? (const __nv_bfloat16*)y[r] : nullptr;
  p.expert_idx = expert_idx; p.src_row_of = src_row_of; p.gate_w = gate_w;
  p.out = (__nv_bfloat16*)out;
  p.residual = (const __nv_bfloat16*)residual;
  p.n_tokens = n_tokens; p.top_k = top_k; p.H = H; p.n_experts = n_experts;
  p.cap_rows = cap_rows;
  p.slot_base = slot_base; p.epoch = epoch;
  p.status = status;
  int grid = resident_grid(4);
  int want = (n_tokens + 7) / 8;
  if (want < grid) grid = want < 1 ? 1 : want;
  moe_combine_kernel<<<grid, 256, 0, STREAM>>>(p);
  return (int)cudaGetLastError();
}
