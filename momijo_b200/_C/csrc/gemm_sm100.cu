// bf16 GEMM on the 5th-generation tensor cores: D[M,N] = op(A) * op(B)^T-style products with
// fp32 accumulation in tensor memory (TMEM), operands staged in shared memory by TMA with a
// 128-byte swizzle, issued by one thread per CTA (tcgen05.mma), persistent over output tiles.
//
// Warp roles inside a 320-thread CTA:
//   warp 0      TMA producer (one lane)
//   warp 1      TMEM allocator + MMA issuer (one lane)
//   warps 2..9  epilogue: tcgen05.ld the accumulator (one output row per thread, two warps per
//               TMEM lane quadrant taking alternate 32-column chunks), apply the fused epilogue
//               (bias / GELU / GELU' / residual / SiLU / scale / accumulate), store bf16 or fp32
// Two accumulators (2 x 256 TMEM columns) let the epilogue of tile i overlap the main loop
// of tile i+1. Tiles are 128 rows tall, or 256 (two MMAs per B stage) for long contractions.
//
// The same kernel also carries the fused communication paths:
//   * gathered operand: extra CTAs pull peer shards over NVLink into local memory and publish
//     per-tile flags that the TMA producer waits on (all-gather -> GEMM);
//   * scattered result: the epilogue stores each row block straight into the memory of the
//     rank that owns it (GEMM -> reduce-scatter, summed by the owner afterwards);
//   * grouped mode for MoE experts (per-tile group table, tile count read from the device).
//
// This replaces the reference's scalar one-thread-per-output kernels
// (legacy/src/momijo/tensor/gpu/runtime.mojo:52-119) and its CPU matmul loops
// (legacy/src/momijo/tensor/broadcast.mojo:1612, legacy/src/momijo/tensor/indexing.mojo:2702).
#include "common.cuh"
#include "gemm_sm100.cuh"

#include <mutex>

namespace mmj {

constexpr int kEpiWarps = 8;
constexpr int kThreads = (2 + kEpiWarps) * 32;  // TMA producer warp, MMA warp, epilogue warps
constexpr int kAStageBytes = kGemmBM * kGemmBK * 2;  // 16 KiB
constexpr int kTmemCols = 512;
constexpr int kAccCols = 256;

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bounded wait until *flag >= want. Returns false on timeout / abort.
__device__ __forceinline__ bool wait_flag_ge(const int* flag, int want, bool sys_scope,
                                             volatile int* abort_flag, int* status, int detail) {
  int v = sys_scope ? ld_acquire_sys(flag) : ld_acquire_gpu(flag);
  if (v >= want) return true;
  uint64_t t0 = 0;  // %globaltimer is slow to read: start the clock only after many polls
  uint32_t it = 0;
  while (true) {
    v = sys_scope ? ld_acquire_sys(flag) : ld_acquire_gpu(flag);
    if (v >= want) return true;
    __nanosleep(32);
    if (((++it) & 0xff) == 0) {
      if (*abort_flag) return false;
      if (status_failed(status)) {
        *abort_flag = 1;
        return false;
      }
      if (t0 == 0) {
        t0 = globaltimer_ns();
        continue;
      }
      if (globaltimer_ns() - t0 > MMJ_WAIT_BUDGET_NS) {
        *abort_flag = 1;
        report(status, kTimeoutFlag, detail);
        return false;
      }
    }
  }
}

struct TileCoord {
  int m_tile, n_tile;
};

// Contraction range of a tile. Plain GEMMs contract over [0, K); in grouped-K mode (expert
// weight gradients) tile t belongs to group g = t / tiles_per_group and contracts over the rows
// [group_k[2g], group_k[2g+1]) of both MN-major operands.
struct KRange {
  int g, tt, k_begin, nk;
};
__device__ __forceinline__ KRange krange_of(int t, int per_group, int num_k, const GemmParams& p) {
  KRange r;
  if (p.groups_k <= 0) {
    r.g = 0; r.tt = t; r.k_begin = 0; r.nk = num_k;
    return r;
  }
  r.g = t / per_group;
  r.tt = t - r.g * per_group;
  r.k_begin = p.group_k[2 * r.g];
  const int k_end = p.group_k[2 * r.g + 1];
  r.nk = (k_end > r.k_begin) ? (k_end - r.k_begin + kGemmBK - 1) / kGemmBK : 0;
  return r;
}

__device__ __forceinline__ TileCoord tile_of(int t, int num_m, int num_n, const GemmParams& p) {
  // n fastest by default: concurrently running CTAs share A rows and sweep B (weights stay in
  // L2). With a gathered B operand the order is m fastest, so that the first waves only need
  // the B tiles that are already local.
  int m_lin, n_lin;
  if (p.flag_mode == 2) {
    n_lin = t / num_m;
    m_lin = t - n_lin * num_m;
  } else if (p.flag_mode == 1 || num_n <= 12) {
    m_lin = t / num_n;
    n_lin = t - m_lin * num_n;
  } else {
    // wide outputs: walk groups of 16 row tiles with n outer / m inner, so that one wave of
    // CTAs covers a roughly square block of tiles and re-reads fewer operand panels from DRAM
    constexpr int kGroupM = 16;
    const int per_group = kGroupM * num_n;
    const int g = t / per_group;
    const int first_m = g * kGroupM;
    const int rows_in_group = min(kGroupM, num_m - first_m);
    const int r = t - g * per_group;
    n_lin = r / rows_in_group;
    m_lin = first_m + (r - n_lin * rows_in_group);
  }
  TileCoord c;
  c.m_tile = m_lin + p.m_tile_rot;
  if (c.m_tile >= num_m) c.m_tile -= num_m;
  c.n_tile = n_lin + p.n_tile_rot;
  if (c.n_tile >= num_n) c.n_tile -= num_n;
  return c;
}

// Byte offset of 16-byte piece `c` (0..3) of row `row` (0..31) in a per-warp staging area of 32 rows x
// 64 bytes. The piece index is XORed with bits 1-2 of the row: the eight lanes of a quarter warp then hit
// eight different 16-byte bank groups both when every lane writes piece c of its own row and when four
// neighbouring lanes read the four pieces of one row (a padded pitch of 80 bytes left the reads of two
// adjacent rows sharing a bank group).
__device__ __forceinline__ int stage_off(int row, int c) {
  return row * 64 + ((c ^ ((row >> 1) & 3)) << 4);
}

// Stores a 32-row x 32-column bf16 chunk (lane = row, v = its 32 columns) through a per-warp
// staging area so that four neighbouring lanes write 64 contiguous bytes of one row: full 32-byte
// sectors per request instead of 32 half-sector pieces. `tile` points at (first row, first column).
__device__ __forceinline__ void staged_store_bf16(uint8_t* st, int lane, const float (&v)[32],
                                                  __nv_bfloat16* tile, long long ld) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 q;
    q.x = pack_bf16x2(v[8 * i + 0], v[8 * i + 1]);
    q.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
    q.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
    q.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
    *reinterpret_cast<uint4*>(st + stage_off(lane, i)) = q;
  }
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rr = 8 * i + (lane >> 2);
    const uint4 q = *reinterpret_cast<const uint4*>(st + stage_off(rr, lane & 3));
    *reinterpret_cast<uint4*>(tile + rr * ld + (lane & 3) * 8) = q;
  }
  __syncwarp();
}

template <bool kOutF32>
__device__ __forceinline__ void epilogue_store_chunk(const GemmParams& p, const uint32_t (&acc)[32],
                                                     int row, int col0, uint8_t* st = nullptr,
                                                     int lane = 0, const uint4* auxq = nullptr) {
  // One thread owns 32 consecutive columns [col0, col0+32) of output row `row`. With `st` set the
  // whole warp is here (32 valid rows, lane = row offset) and full chunks leave through it. `auxq`:
  // the chunk's 32 aux values, already loaded by the caller (full chunks only).
  const int epi = p.epi;
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(acc[i]);

  const bool full = p.vec_ok && (col0 + 32 <= p.N);
  if (epi & kEpiBias) {
    const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(p.bias) + col0;
    if (full) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 q = __ldg(reinterpret_cast<const uint4*>(b) + i);
        float2 f0 = unpack_bf16x2(q.x), f1 = unpack_bf16x2(q.y), f2 = unpack_bf16x2(q.z),
               f3 = unpack_bf16x2(q.w);
        v[8 * i + 0] += f0.x; v[8 * i + 1] += f0.y; v[8 * i + 2] += f1.x; v[8 * i + 3] += f1.y;
        v[8 * i + 4] += f2.x; v[8 * i + 5] += f2.y; v[8 * i + 6] += f3.x; v[8 * i + 7] += f3.y;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N) v[i] += __bfloat162float(b[i]);
    }
  }
  if (epi & kEpiGelu) {
    __nv_bfloat16* d2 = reinterpret_cast<__nv_bfloat16*>(p.D2) + (long long)row * p.ldd2 + col0;
    if (full && st != nullptr) {
      staged_store_bf16(st, lane, v, d2 - (long long)lane * p.ldd2, p.ldd2);
    } else if (full) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 q;
        q.x = pack_bf16x2(v[8 * i + 0], v[8 * i + 1]);
        q.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
        q.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
        q.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
        reinterpret_cast<uint4*>(d2)[i] = q;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N) d2[i] = __float2bfloat16(v[i]);
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
  }
  if (epi & kEpiSilu) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = v[i] / (1.0f + __expf(-v[i]));
  }
  if (epi & (kEpiDGelu | kEpiAddAux | kEpiMulAux)) {
    const __nv_bfloat16* a =
        reinterpret_cast<const __nv_bfloat16*>(p.aux) + (long long)row * p.ldaux + col0;
    float x[32];
    if (full) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 q = (auxq != nullptr) ? auxq[i] : reinterpret_cast<const uint4*>(a)[i];
        float2 f0 = unpack_bf16x2(q.x), f1 = unpack_bf16x2(q.y), f2 = unpack_bf16x2(q.z),
               f3 = unpack_bf16x2(q.w);
        x[8 * i + 0] = f0.x; x[8 * i + 1] = f0.y; x[8 * i + 2] = f1.x; x[8 * i + 3] = f1.y;
        x[8 * i + 4] = f2.x; x[8 * i + 5] = f2.y; x[8 * i + 6] = f3.x; x[8 * i + 7] = f3.y;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) x[i] = (col0 + i < p.N) ? __bfloat162float(a[i]) : 0.f;
    }
    if (epi & kEpiDGelu) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] *= gelu_tanh_grad(x[i]);
    } else if (epi & kEpiMulAux) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] *= x[i];
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] += x[i];
    }
  }
  if (epi & kEpiRowScale) {
    const float s = p.row_scale[row];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] *= s;
  }

  // Destination row: local, or the owner's staging slot for the reduce-scatter epilogue.
  long long off;
  void* base = p.D;
  if (epi & kEpiScatterPeers) {
    int owner = row / p.rows_per_rank;
    int lrow = row - owner * p.rows_per_rank;
    base = p.peer_D[owner];
    off = (long long)p.rank * p.slot_stride + (long long)lrow * p.ldd + col0;
  } else {
    off = (long long)row * p.ldd + col0;
  }

  if (kOutF32) {
    float* d = reinterpret_cast<float*>(base) + off;
    if (full) {
      if (epi & kEpiAccumulate) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float4 o = reinterpret_cast<float4*>(d)[i];
          v[4 * i + 0] += o.x; v[4 * i + 1] += o.y; v[4 * i + 2] += o.z; v[4 * i + 3] += o.w;
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
        reinterpret_cast<float4*>(d)[i] =
            make_float4(v[4 * i + 0], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N) d[i] = (epi & kEpiAccumulate) ? d[i] + v[i] : v[i];
    }
  } else {
    __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(base) + off;
    if (full && st != nullptr && !(epi & (kEpiAccumulate | kEpiScatterPeers))) {
      staged_store_bf16(st, lane, v, d - (long long)lane * p.ldd, p.ldd);
    } else if (full) {
      if (epi & kEpiAccumulate) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 q = reinterpret_cast<uint4*>(d)[i];
          float2 f0 = unpack_bf16x2(q.x), f1 = unpack_bf16x2(q.y), f2 = unpack_bf16x2(q.z),
                 f3 = unpack_bf16x2(q.w);
          v[8 * i + 0] += f0.x; v[8 * i + 1] += f0.y; v[8 * i + 2] += f1.x; v[8 * i + 3] += f1.y;
          v[8 * i + 4] += f2.x; v[8 * i + 5] += f2.y; v[8 * i + 6] += f3.x; v[8 * i + 7] += f3.y;
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 q;
        q.x = pack_bf16x2(v[8 * i + 0], v[8 * i + 1]);
        q.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
        q.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
        q.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
        reinterpret_cast<uint4*>(d)[i] = q;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N) {
          float o = (epi & kEpiAccumulate) ? __bfloat162float(d[i]) : 0.f;
          d[i] = __float2bfloat16(v[i] + o);
        }
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA,
                         const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzled tiles need 1024-byte aligned bases.
  // (offset arithmetic on the __shared__ symbol, not an integer round trip, so that the compiler
  // keeps the shared address space and emits shared rather than generic loads and stores)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ __align__(8) uint64_t full_bar[kGemmMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kGemmMaxStages];
  __shared__ __align__(8) uint64_t tfull_bar[2];
  __shared__ __align__(8) uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  // per-warp staging for the transposing stores: 32 rows x 64 bytes, pieces swizzled (stage_off)
  __shared__ __align__(16) uint8_t epi_stage[kEpiWarps][32 * 64];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int gemm_ctas = (p.gemm_ctas > 0) ? p.gemm_ctas : (int)gridDim.x;

  // ---------------- communication CTAs: pull peer shards, publish per-tile flags ----------
  // One thread per CTA drives bulk asynchronous copies (peer memory -> shared memory ->
  // local memory) through a ring of 32 KiB buffers, so that ~190 KiB per CTA stay in flight
  // over NVLink without occupying the other threads. No multicast is involved.
  if ((int)blockIdx.x >= gemm_ctas) {
    constexpr int kNBuf = 6;
    constexpr int kBufBytes = 32 * 1024;
    if (threadIdx.x == 0) {
      abort_flag = 0;
      for (int b = 0; b < kNBuf; ++b) mbar_init(&full_bar[b], 1);
      mbar_fence_init();
      const int n_comm = (int)gridDim.x - gemm_ctas;
      const int cid = (int)blockIdx.x - gemm_ctas;
      const int ntiles = (int)((p.gather_total_bytes + p.tile_bytes - 1) / p.tile_bytes);
      const int rot = p.comm_rot;
      uint32_t issued = 0, drained = 0;  // chunk counters over the ring
      bool ok = true;
      for (int i = cid; i < ntiles && ok; i += n_comm) {
        int t = i + rot;  // same visiting order as the GEMM CTAs consume tiles
        if (t >= ntiles) t -= ntiles;
        long long lo = (long long)t * p.tile_bytes;
        long long hi = lo + p.tile_bytes;
        if (hi > p.gather_total_bytes) hi = p.gather_total_bytes;
        // a tile may straddle shard boundaries: copy it owner by owner
        while (lo < hi && ok) {
          const long long abs_off = p.gather_flat_off + lo;
          const int owner = (int)(abs_off / p.shard_bytes);
          long long seg_hi = (long long)(owner + 1) * p.shard_bytes - p.gather_flat_off;
          if (seg_hi > hi) seg_hi = hi;
          if ((owner != p.rank || p.src_compact) && owner < p.world) {
            if (p.peer_ready != nullptr && owner != p.rank)
              ok = wait_flag_ge(p.peer_ready + owner, p.ready_epoch, true, &abort_flag, p.status,
                                100 + owner);
            if (!ok) break;
            const long long nbytes = seg_hi - lo;
            const uint8_t* src = reinterpret_cast<const uint8_t*>(p.peer_src[owner]) +
                                 (p.src_compact ? (abs_off - (long long)owner * p.shard_bytes) : lo);
            uint8_t* dst = reinterpret_cast<uint8_t*>(p.gather_dst) + lo;
            const int nchunks = (int)((nbytes + kBufBytes - 1) / kBufBytes);
            int next_load = 0;
            for (int c = 0; c < nchunks && ok; ++c) {
              // keep up to kNBuf loads in flight
              while (next_load < nchunks && issued - drained < (uint32_t)kNBuf) {
                const int b = issued % kNBuf;
                const long long co = (long long)next_load * kBufBytes;
                const uint32_t sz =
                    (uint32_t)((nbytes - co < kBufBytes) ? (nbytes - co) : kBufBytes);
                mbar_expect_tx(&full_bar[b], sz);
                asm volatile(
                    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                    ::"r"(smem_u32(smem + (size_t)b * kBufBytes)), "l"(src + co), "r"(sz),
                    "r"(smem_u32(&full_bar[b]))
                    : "memory");
                ++issued;
                ++next_load;
              }
              const int b = drained % kNBuf;
              const uint32_t par = (drained / kNBuf) & 1u;
              if (!mbar_wait(&full_bar[b], par, &abort_flag, p.status, kTimeoutFull, 1000 + c)) {
                ok = false;
                break;
              }
              const long long co = (long long)c * kBufBytes;
              const uint32_t sz = (uint32_t)((nbytes - co < kBufBytes) ? (nbytes - co) : kBufBytes);
              asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst + co),
                           "r"(smem_u32(smem + (size_t)b * kBufBytes)), "r"(sz)
                           : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
              // the buffer may be refilled once the store has read it
              asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
              ++drained;
            }
            // all bytes of this piece written before the tile's flag is published
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
          }
          lo = seg_hi;
        }
        if (!ok) break;
        asm volatile("fence.proxy.async;" ::: "memory");
        __threadfence();
        st_release_gpu(p.flags_rw + t, p.ready_epoch);
      }
      // never leave with loads in flight into this CTA's shared memory
      while (drained < issued) {
        const int b = drained % kNBuf;
        const uint32_t par = (drained / kNBuf) & 1u;
        int local_abort = 0;
        if (!mbar_wait(&full_bar[b], par, &local_abort, p.status, kTimeoutFull, 2000)) break;
        ++drained;
      }
    }
    return;
  }

  // ---------------- GEMM CTAs --------------------------------------------------------------
  const int bn = p.bn;
  const int stages = p.stages;
  const int b_stage_bytes = bn * kGemmBK * 2;
  // Tall tiles (bm2): 256 rows per tile as two 128-row sub-tiles that share each B stage, which
  // halves the B bytes pulled from L2 per FLOP. With bn = 256 the two accumulators take all 512
  // TMEM columns, so the epilogue of a tile no longer overlaps the next tile's main loop.
  const int subs = p.bm2 ? 2 : 1;
  const int bm = kGemmBM * subs;
  const int a_bytes = kAStageBytes * subs;
  const int stage_bytes = a_bytes + b_stage_bytes;
  const int n_acc = (subs * bn > kAccCols) ? 1 : 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], kEpiWarps);
    }
    abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  // everything above touched no global memory: it may run under the previous kernel's tail
  pdl_wait();
  pdl_trigger();

  const int num_m = (p.num_m_tiles_dev != nullptr) ? *p.num_m_tiles_dev
                                                   : (p.M + bm - 1) / bm;
  const int num_n = (p.N + bn - 1) / bn;
  const int num_k = (p.K + kGemmBK - 1) / kGemmBK;
  const int per_group = num_m * num_n;
  const int num_tiles = (p.groups_k > 0) ? p.groups_k * per_group : per_group;

  if (num_k > 0 || p.groups_k > 0) {
    if (warp == 0) {
      // ======================= TMA producer =======================
      if (lane == 0) {
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gemm_ctas) {
          const KRange kr = krange_of(t, per_group, num_k, p);
          const TileCoord tc = tile_of(kr.tt, num_m, num_n, p);
          const int m0 = tc.m_tile * bm;
          const int n0 = tc.n_tile * bn;
          const int g = (p.tile_group != nullptr) ? p.tile_group[tc.m_tile] : 0;
          const int b_row_base = g * p.b_group_rows;
          if (p.flag_mode == 1) {
            // flags are per 128-row granule of the gathered operand: a tall tile needs two
            const int n_gran = (p.M + kGemmBM - 1) / kGemmBM;
            for (int sub = 0; sub < subs && ok; ++sub) {
              const int gt = tc.m_tile * subs + sub;
              if (gt < n_gran)
                ok = wait_flag_ge(p.ready_flags + gt, p.ready_epoch, false, &abort_flag, p.status, gt);
            }
            asm volatile("fence.proxy.async;" ::: "memory");
          } else if (p.flag_mode == 2) {
            ok = wait_flag_ge(p.ready_flags + tc.n_tile, p.ready_epoch, false, &abort_flag,
                              p.status, tc.n_tile);
            asm volatile("fence.proxy.async;" ::: "memory");
          }
          if (!ok) break;
          for (int kb = 0; kb < kr.nk; ++kb) {
            if (!mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag, p.status, kTimeoutEmpty, kb)) {
              ok = false;
              break;
            }
            uint8_t* sA = smem + (size_t)s * stage_bytes;
            uint8_t* sB = sA + a_bytes;
            mbar_expect_tx(&full_bar[s], (uint32_t)stage_bytes);
            const int k0 = kr.k_begin + kb * kGemmBK;
            for (int sub = 0; sub < subs; ++sub) {
              uint8_t* sAs = sA + sub * kAStageBytes;
              const int ms = m0 + sub * kGemmBM;
              if (!p.a_mn) {
                tma_load_2d(sAs, &tmA, &full_bar[s], k0, ms);
              } else {
                tma_load_2d(sAs, &tmA, &full_bar[s], ms, k0);
                tma_load_2d(sAs + 8192, &tmA, &full_bar[s], ms + 64, k0);
              }
            }
            if (!p.b_mn) {
              tma_load_2d(sB, &tmB, &full_bar[s], k0, b_row_base + n0);
            } else {
              for (int j = 0; j < bn / 64; ++j)
                tma_load_2d(sB + j * 8192, &tmB, &full_bar[s], n0 + 64 * j, b_row_base + k0);
            }
            if (++s == stages) { s = 0; ph ^= 1; }
          }
        }
      }
    } else if (warp == 1) {
      // ======================= MMA issuer =======================
      if (lane == 0) {
        const uint32_t idesc = make_idesc_bf16(kGemmBM, bn, p.a_mn, p.b_mn);
        const uint32_t a_lbo = p.a_mn ? 8192u : 16u;
        const uint32_t b_lbo = p.b_mn ? 8192u : 16u;
        const uint32_t a_kstep = p.a_mn ? 2048u : 32u;
        const uint32_t b_kstep = p.b_mn ? 2048u : 32u;
        int s = 0;
        uint32_t ph = 0;
        int acc = 0;
        uint32_t acc_ph = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gemm_ctas) {
          const KRange kr = krange_of(t, per_group, num_k, p);
          if (kr.nk == 0) continue;  // empty contraction: the epilogue writes zeros on its own
          if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1, &abort_flag, p.status, kTimeoutTmemEmpty,
                         t)) {
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * kAccCols);
          const uint32_t d_tmem1 = d_tmem + (uint32_t)bn;  // second sub-tile of a tall tile
          for (int kb = 0; kb < kr.nk; ++kb) {
            if (!mbar_wait(&full_bar[s], ph, &abort_flag, p.status, kTimeoutFull, kb)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t a_base = smem_u32(smem + (size_t)s * stage_bytes);
            const uint32_t b_base = a_base + (uint32_t)a_bytes;
#pragma unroll
            for (int k = 0; k < kGemmBK / 16; ++k) {
              const uint64_t da = make_smem_desc(a_base + k * a_kstep, a_lbo, 1024);
              const uint64_t db = make_smem_desc(b_base + k * b_kstep, b_lbo, 1024);
              umma_bf16_ss(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
              if (subs == 2) {
                const uint64_t da1 = make_smem_desc(a_base + kAStageBytes + k * a_kstep, a_lbo, 1024);
                umma_bf16_ss(d_tmem1, da1, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
              }
            }
            umma_commit(&empty_bar[s]);  // frees the smem stage once these MMAs retire
            if (++s == stages) { s = 0; ph ^= 1; }
          }
          if (!ok) break;
          umma_commit(&tfull_bar[acc]);  // accumulator complete
          if (++acc == n_acc) { acc = 0; acc_ph ^= 1; }
        }
      }
    } else {
      // ======================= epilogue warps =======================
      // Eight epilogue warps: two per TMEM lane quadrant (a warp reaches the 32 lanes of quadrant
      // warp % 4 only), taking alternate 32-column chunks. With four warps the fused GELU / GELU'
      // epilogues of the K = 768 products took longer than the next tile's main loop.
      const int quad = warp & 3;
      const int chalf = (warp - 2) >> 2;
      int acc = 0;
      uint32_t acc_ph = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gemm_ctas) {
        const KRange kr = krange_of(t, per_group, num_k, p);
        const TileCoord tc = tile_of(kr.tt, num_m, num_n, p);
        const int m0 = tc.m_tile * bm;
        const int n0 = tc.n_tile * bn;
        const int out_row0 = kr.g * p.M;  // grouped-K: group g writes rows [g*M, (g+1)*M)
        if (kr.nk == 0) {
          // nothing to contract (an expert without tokens): the result is zero
          for (int sub = 0; sub < subs; ++sub) {
          const int zrow = m0 + sub * kGemmBM + quad * 32 + lane;
          if (zrow < p.M) {
            uint32_t z[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) z[i] = 0u;
            for (int c = chalf; c < bn / 32; c += 2) {
              const int col0 = n0 + c * 32;
              if (col0 < p.N) {
                if (p.epi & kEpiOutF32)
                  epilogue_store_chunk<true>(p, z, zrow + out_row0, col0);
                else
                  epilogue_store_chunk<false>(p, z, zrow + out_row0, col0);
              }
            }
          }
          }
          continue;
        }
        if (!mbar_wait_warp(&tfull_bar[acc], acc_ph, &abort_flag, p.status, kTimeoutTmemFull, t)) break;
        tc_fence_after();
        for (int sub = 0; sub < subs; ++sub) {
          const int row = m0 + sub * kGemmBM + quad * 32 + lane;
          const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) +
                                 (uint32_t)(acc * kAccCols + sub * bn);
          for (int c = chalf; c < bn / 32; c += 2) {
            uint32_t r[32];
            tmem_ld_32x32(t_row + (uint32_t)(c * 32), r);
            tmem_ld_wait();
            const int col0 = n0 + c * 32;
            if ((p.epi & kEpiScatterPeers) && p.vec_ok && col0 + 32 <= p.N) {
              // Stores into a peer's memory travel over NVLink: transpose the chunk through shared
              // memory so that four neighbouring lanes write 64 contiguous bytes of one row (one
              // thread per row would send 16-byte pieces).
              uint8_t* st = epi_stage[warp - 2];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 q;
                q.x = pack_bf16x2(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]));
                q.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
                q.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
                q.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
                *reinterpret_cast<uint4*>(st + stage_off(lane, i)) = q;
              }
              __syncwarp();
              const int row_base = m0 + sub * kGemmBM + quad * 32;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int rr = 8 * i + (lane >> 2);
                const uint4 q = *reinterpret_cast<const uint4*>(st + stage_off(rr, lane & 3));
                const int grow = row_base + rr;
                if (grow < p.M) {
                  const int owner = grow / p.rows_per_rank;
                  const int lrow = grow - owner * p.rows_per_rank;
                  __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(p.peer_D[owner]) +
                                     (long long)p.rank * p.slot_stride + (long long)lrow * p.ldd + col0 +
                                     (lane & 3) * 8;
                  *reinterpret_cast<uint4*>(d) = q;
                }
              }
              __syncwarp();
            } else if (row < p.M && col0 < p.N) {
              if (p.epi & kEpiOutF32)
                epilogue_store_chunk<true>(p, r, row + out_row0, col0);
              else
                epilogue_store_chunk<false>(
                    p, r, row + out_row0, col0,
                    (m0 + sub * kGemmBM + quad * 32 + 32 <= p.M) ? epi_stage[warp - 2] : nullptr, lane);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[acc]);
        if (++acc == n_acc) { acc = 0; acc_ph ^= 1; }
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// CTA-pair variant (cta_group::2) for plain products: two CTAs of a cluster own one 256 x 256 tile.
// Each CTA stages its own 128 rows of A and its own 128-column half of B (32 KiB per 64-deep K
// block instead of 48 KiB for a 128 x 256 tile on one CTA: a third less traffic from L2 into shared
// memory per FLOP), keeps 128 x 256 of the accumulator in its own TMEM (two accumulators, so the
// epilogue still overlaps the next main loop) and stores its own rows. The rank-0 CTA issues the
// MMAs for the pair; both CTAs' loads are credited to rank 0's "full" barrier, the MMA's commits
// release the stage in both CTAs, and both CTAs' epilogue warps arrive on rank 0's "accumulator
// free" barrier. No load uses multicast.
// ---------------------------------------------------------------------------------------------
constexpr int kPairBN = 256;
constexpr int kPairStageBytes = kAStageBytes + (kPairBN / 2) * kGemmBK * 2;  // 32 KiB

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ __align__(8) uint64_t full_bar[kGemmMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kGemmMaxStages];
  __shared__ __align__(8) uint64_t tfull_bar[2];
  __shared__ __align__(8) uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ __align__(16) uint8_t epi_stage[kEpiWarps][32 * 64];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = (int)blockIdx.x >> 1;
  const int num_pairs = (int)gridDim.x >> 1;
  const int stages = p.stages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 2 * kEpiWarps);  // epilogue warps of both CTAs (used on rank 0)
    }
    abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(&tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  pdl_wait();  // nothing above touched global memory
  pdl_trigger();

  const int num_m = (p.M + 2 * kGemmBM - 1) / (2 * kGemmBM);
  const int num_n = (p.N + kPairBN - 1) / kPairBN;
  const int num_k = (p.K + kGemmBK - 1) / kGemmBK;
  const int per_group = num_m * num_n;
  const int num_tiles = (p.groups_k > 0) ? p.groups_k * per_group : per_group;

  if (num_k > 0 || p.groups_k > 0) {
    if (warp == 0) {
      // ======================= TMA producer (both CTAs) =======================
      if (lane == 0) {
        const uint32_t full0 = mapa_shared(smem_u32(&full_bar[0]), 0);  // rank 0's barriers
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += num_pairs) {
          const KRange kr = krange_of(t, per_group, num_k, p);
          const TileCoord tc = tile_of(kr.tt, num_m, num_n, p);
          const int m0 = tc.m_tile * 2 * kGemmBM + (int)rank * kGemmBM;
          const int n0 = tc.n_tile * kPairBN + (int)rank * (kPairBN / 2);
          for (int kb = 0; kb < kr.nk; ++kb) {
            if (!mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag, p.status, kTimeoutEmpty, kb)) {
              ok = false;
              break;
            }
            uint8_t* sA = smem + (size_t)s * kPairStageBytes;
            uint8_t* sB = sA + kAStageBytes;
            if (leader) mbar_expect_tx(&full_bar[s], 2u * (uint32_t)kPairStageBytes);
            const uint32_t fb = full0 + (uint32_t)(s * sizeof(uint64_t));
            const int k0 = kr.k_begin + kb * kGemmBK;
            if (!p.a_mn) {
              tma_load_2d_pair(sA, &tmA, fb, k0, m0);
            } else {
              tma_load_2d_pair(sA, &tmA, fb, m0, k0);
              tma_load_2d_pair(sA + 8192, &tmA, fb, m0 + 64, k0);
            }
            if (!p.b_mn) {
              tma_load_2d_pair(sB, &tmB, fb, k0, n0);
            } else {
              tma_load_2d_pair(sB, &tmB, fb, n0, k0);
              tma_load_2d_pair(sB + 8192, &tmB, fb, n0 + 64, k0);
            }
            if (++s == stages) { s = 0; ph ^= 1; }
          }
        }
      }
    } else if (warp == 1) {
      // ======================= MMA issuer (rank 0 only) =======================
      if (lane == 0 && leader) {
        const uint32_t idesc = make_idesc_bf16(2 * kGemmBM, kPairBN, p.a_mn, p.b_mn);
        const uint32_t a_lbo = p.a_mn ? 8192u : 16u;
        const uint32_t b_lbo = p.b_mn ? 8192u : 16u;
        const uint32_t a_kstep = p.a_mn ? 2048u : 32u;
        const uint32_t b_kstep = p.b_mn ? 2048u : 32u;
        const uint32_t empty_own = smem_u32(&empty_bar[0]);
        const uint32_t empty_peer = mapa_shared(empty_own, 1);
        const uint32_t tfull_own = smem_u32(&tfull_bar[0]);
        const uint32_t tfull_peer = mapa_shared(tfull_own, 1);
        const uint32_t empty_own_c = mapa_shared(empty_own, 0);
        const uint32_t tfull_own_c = mapa_shared(tfull_own, 0);
        int s = 0;
        uint32_t ph = 0;
        int acc = 0;
        uint32_t acc_ph = 0;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += num_pairs) {
          const KRange kr = krange_of(t, per_group, num_k, p);
          if (kr.nk == 0) continue;  // empty contraction: the epilogues write zeros on their own
          if (!mbar_wait(&tempty_bar[acc], acc_ph ^ 1, &abort_flag, p.status, kTimeoutTmemEmpty,
                         t)) {
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * kAccCols);
          for (int kb = 0; kb < kr.nk; ++kb) {
            if (!mbar_wait(&full_bar[s], ph, &abort_flag, p.status, kTimeoutFull, kb)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t a_base = smem_u32(smem + (size_t)s * kPairStageBytes);
            const uint32_t b_base = a_base + (uint32_t)kAStageBytes;
#pragma unroll
            for (int k = 0; k < kGemmBK / 16; ++k) {
              const uint64_t da = make_smem_desc(a_base + k * a_kstep, a_lbo, 1024);
              const uint64_t db = make_smem_desc(b_base + k * b_kstep, b_lbo, 1024);
              umma_bf16_ss_pair(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
            // the stage is free in both CTAs once these MMAs retire
            umma_commit_pair(empty_own_c + (uint32_t)(s * sizeof(uint64_t)));
            umma_commit_pair(empty_peer + (uint32_t)(s * sizeof(uint64_t)));
            if (++s == stages) { s = 0; ph ^= 1; }
          }
          if (!ok) break;
          umma_commit_pair(tfull_own_c + (uint32_t)(acc * sizeof(uint64_t)));
          umma_commit_pair(tfull_peer + (uint32_t)(acc * sizeof(uint64_t)));
          if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
      }
    } else {
      // ======================= epilogue warps (both CTAs) =======================
      const int quad = warp & 3;
      const int chalf = (warp - 2) >> 2;
      const uint32_t tempty0 = mapa_shared(smem_u32(&tempty_bar[0]), 0);
      int acc = 0;
      uint32_t acc_ph = 0;
      for (int t = pair; t < num_tiles; t += num_pairs) {
        const KRange kr = krange_of(t, per_group, num_k, p);
        const TileCoord tc = tile_of(kr.tt, num_m, num_n, p);
        const int m0 = tc.m_tile * 2 * kGemmBM + (int)rank * kGemmBM;
        const int n0 = tc.n_tile * kPairBN;
        const int out_row0 = kr.g * p.M;  // grouped-K: group g writes rows [g*M, (g+1)*M)
        if (kr.nk == 0) {
          const int zrow = m0 + quad * 32 + lane;
          if (zrow < p.M) {
            uint32_t z[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) z[i] = 0u;
            for (int c = chalf; c < kPairBN / 32; c += 2) {
              const int col0 = n0 + c * 32;
              if (col0 < p.N) {
                if (p.epi & kEpiOutF32)
                  epilogue_store_chunk<true>(p, z, zrow + out_row0, col0);
                else
                  epilogue_store_chunk<false>(p, z, zrow + out_row0, col0);
              }
            }
          }
          continue;
        }
        if (!mbar_wait_warp(&tfull_bar[acc], acc_ph, &abort_flag, p.status, kTimeoutTmemFull, t)) break;
        tc_fence_after();
        const int row = m0 + quad * 32 + lane;
        const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * kAccCols);
        uint8_t* st = (m0 + quad * 32 + 32 <= p.M) ? epi_stage[warp - 2] : nullptr;
        // The aux operand of the GELU' / add / multiply epilogues is requested one chunk ahead, so that
        // its latency hides behind the previous chunk instead of following every TMEM read.
        const bool has_aux = (p.epi & (kEpiDGelu | kEpiAddAux | kEpiMulAux)) != 0 && p.vec_ok && row < p.M;
        const __nv_bfloat16* aux_row =
            reinterpret_cast<const __nv_bfloat16*>(p.aux) + (long long)(row + out_row0) * p.ldaux;
        uint4 aq[4], aq_next[4];
        bool aq_ok = false, aq_next_ok = false;
#pragma unroll
        for (int i = 0; i < 4; ++i) aq_next[i] = make_uint4(0u, 0u, 0u, 0u);
        if (has_aux && n0 + chalf * 32 + 32 <= p.N) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            aq_next[i] = reinterpret_cast<const uint4*>(aux_row + n0 + chalf * 32)[i];
          aq_next_ok = true;
        }
        for (int c = chalf; c < kPairBN / 32; c += 2) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + (uint32_t)(c * 32), r);
#pragma unroll
          for (int i = 0; i < 4; ++i) aq[i] = aq_next[i];
          aq_ok = aq_next_ok;
          aq_next_ok = false;
          const int ncol0 = n0 + (c + 2) * 32;
          if (has_aux && c + 2 < kPairBN / 32 && ncol0 + 32 <= p.N) {
#pragma unroll
            for (int i = 0; i < 4; ++i) aq_next[i] = reinterpret_cast<const uint4*>(aux_row + ncol0)[i];
            aq_next_ok = true;
          }
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (row < p.M && col0 < p.N) {
            if (p.epi & kEpiOutF32)
              epilogue_store_chunk<true>(p, r, row + out_row0, col0, nullptr, 0, aq_ok ? aq : nullptr);
            else
              epilogue_store_chunk<false>(p, r, row + out_row0, col0, st, lane, aq_ok ? aq : nullptr);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tempty0 + (uint32_t)(acc * sizeof(uint64_t)));
        if (++acc == 2) { acc = 0; acc_ph ^= 1; }
      }
    }
  }

  // ---------------- teardown: neither CTA leaves (or frees TMEM) while its peer may still signal it
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(f);
  });
  return fn;
}

// The driver call below needs the primary context to be current on the calling thread; threads
// that have only been handed a device ordinal (e.g. autograd workers) bind it on first use.
void ensure_context() {
  static thread_local bool ready = false;
  if (!ready) {
    cudaFree(0);
    ready = true;
  }
}

// 2-D bf16 tensor map: `inner` contiguous elements, `outer` rows `row_stride_elems` apart.
// A descriptor is a pure function of (address, extents, stride, box), and a training step asks for the
// same few hundred of them every iteration, so encoded maps are kept in a small per-thread
// direct-mapped cache instead of calling into the driver twice per GEMM launch.
struct TmapKey {
  const void* base;
  uint64_t inner, outer, stride;
  uint32_t box_inner, box_outer;
  bool operator==(const TmapKey& o) const {
    return base == o.base && inner == o.inner && outer == o.outer && stride == o.stride &&
           box_inner == o.box_inner && box_outer == o.box_outer;
  }
};
struct TmapSlot {
  TmapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int kTmapCacheSlots = 1024;

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_elems, uint32_t box_inner, uint32_t box_outer) {
  static thread_local TmapSlot* cache = nullptr;
  if (cache == nullptr) cache = new TmapSlot[kTmapCacheSlots]();
  const TmapKey key{base, inner, outer, row_stride_elems, box_inner, box_outer};
  uint64_t h = (uint64_t)(uintptr_t)base * 0x9E3779B97F4A7C15ull;
  h ^= (inner * 0xC2B2AE3D27D4EB4Full) ^ (outer * 0x165667B19E3779F9ull) ^ (row_stride_elems << 17) ^
       ((uint64_t)box_inner << 40) ^ ((uint64_t)box_outer << 48);
  TmapSlot& slot = cache[(h >> 20) & (kTmapCacheSlots - 1)];
  if (slot.used && slot.key == key) {
    *out = slot.map;
    return 0;
  }
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  ensure_context();
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return (int)r;
  slot.key = key;
  slot.map = *out;
  slot.used = true;
  return 0;
}

static int g_sm_count = 0;
static int sm_count() {
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (g_sm_count <= 0) g_sm_count = 148;
  }
  return g_sm_count;
}

static bool g_attr_set = false;
static int g_max_dyn_smem = 0;

int launch_gemm(GemmParams& p, const void* A, long long lda, long long a_rows, const void* B,
                long long ldb, long long b_rows, int comm_ctas, cudaStream_t stream) {
  if (p.M <= 0 || p.N <= 0) return 0;
  if ((lda % 8) != 0 || (ldb % 8) != 0) return -2;
  {
    // 16-byte vector accesses in the epilogue need aligned bases and leading dimensions.
    const int out_elems = (p.epi & kEpiOutF32) ? 4 : 8;
    bool ok = (p.ldd % out_elems == 0) && (((uintptr_t)p.D & 15) == 0);
    if (p.epi & kEpiScatterPeers)
      for (int r = 0; r < p.world; ++r) ok = ok && (((uintptr_t)p.peer_D[r] & 15) == 0);
    if (p.epi & kEpiScatterPeers) ok = ok && (p.slot_stride % out_elems == 0);
    if (p.epi & kEpiBias) ok = ok && (((uintptr_t)p.bias & 15) == 0);
    if (p.epi & kEpiGelu) ok = ok && (p.ldd2 % 8 == 0) && (((uintptr_t)p.D2 & 15) == 0);
    if (p.epi & (kEpiDGelu | kEpiAddAux | kEpiMulAux))
      ok = ok && (p.ldaux % 8 == 0) && (((uintptr_t)p.aux & 15) == 0);
    p.vec_ok = ok ? 1 : 0;
  }
  if (((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return -3;
  if (p.bn != 64 && p.bn != 128 && p.bn != 256) return -4;
  CUtensorMap tmA, tmB;
  int rc;
  // A: K-major [a_rows(M), K] or MN-major [a_rows(K), M]
  if (!p.a_mn)
    rc = make_tmap_bf16_2d(&tmA, A, (uint64_t)p.K, (uint64_t)a_rows, (uint64_t)lda, 64, 128);
  else
    rc = make_tmap_bf16_2d(&tmA, A, (uint64_t)p.M, (uint64_t)a_rows, (uint64_t)lda, 64, 64);
  if (rc) return rc;
  if (!p.b_mn)
    rc = make_tmap_bf16_2d(&tmB, B, (uint64_t)p.K, (uint64_t)b_rows, (uint64_t)ldb, 64,
                           (uint32_t)p.bn);
  else
    rc = make_tmap_bf16_2d(&tmB, B, (uint64_t)p.N, (uint64_t)b_rows, (uint64_t)ldb, 64, 64);
  if (rc) return rc;

  if (p.bm2 && p.tile_group != nullptr) return -5;
  const int stage_bytes = kAStageBytes * (p.bm2 ? 2 : 1) + p.bn * kGemmBK * 2;
  int stages = (200 * 1024) / stage_bytes;
  if (stages > kGemmMaxStages) stages = kGemmMaxStages;
  p.stages = stages;
  const int smem_bytes = stages * stage_bytes + 1024;
  if (!g_attr_set) {
    // static shared memory (barriers, the scatter staging) counts against the same 227 KB
    cudaFuncAttributes fa;
    cudaError_t e = cudaFuncGetAttributes(&fa, gemm_bf16_tcgen05_kernel);
    if (e != cudaSuccess) return (int)e;
    g_max_dyn_smem = 232448 - (int)fa.sharedSizeBytes;
    e = cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             g_max_dyn_smem);
    if (e != cudaSuccess) return (int)e;
    g_attr_set = true;
  }
  if (smem_bytes > g_max_dyn_smem) return -6;
  const int bm = kGemmBM * (p.bm2 ? 2 : 1);
  const int num_m = (p.M + bm - 1) / bm;
  const int num_n = (p.N + p.bn - 1) / p.bn;
  long long tiles = (long long)num_m * num_n;
  if (p.groups_k > 0) tiles *= p.groups_k;
  int gemm_ctas = sm_count() - comm_ctas;
  if (gemm_ctas < 1) gemm_ctas = 1;
  if (tiles < gemm_ctas) gemm_ctas = (int)tiles;
  p.gemm_ctas = gemm_ctas;
  if (comm_ctas == 0 && p.flag_mode == 0) {
    // plain product: set-up may overlap the previous kernel's tail
    cudaError_t e = launch_pdl(gemm_bf16_tcgen05_kernel, dim3(gemm_ctas), dim3(kThreads), (size_t)smem_bytes,
                               stream, tmA, tmB, p);
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
  }
  // products fused with a collective wait on other ranks: ordinary stream order
  gemm_bf16_tcgen05_kernel<<<gemm_ctas + comm_ctas, kThreads, smem_bytes, stream>>>(tmA, tmB, p);
  return (int)cudaGetLastError();
}

// Pair kernel launcher: plain products only (no flags, groups, gathered or scattered operands).
static int g_pair_max_dyn = 0;
static int g_pair_clusters = 0;

int launch_gemm_pair(GemmParams& p, const void* A, long long lda, long long a_rows, const void* B,
                     long long ldb, long long b_rows, cudaStream_t stream) {
  if (p.M <= 0 || p.N <= 0) return 0;
  if ((lda % 8) != 0 || (ldb % 8) != 0) return -2;
  if (p.epi & kEpiScatterPeers) return -7;
  {
    const int out_elems = (p.epi & kEpiOutF32) ? 4 : 8;
    bool ok = (p.ldd % out_elems == 0) && (((uintptr_t)p.D & 15) == 0);
    if (p.epi & kEpiBias) ok = ok && (((uintptr_t)p.bias & 15) == 0);
    if (p.epi & kEpiGelu) ok = ok && (p.ldd2 % 8 == 0) && (((uintptr_t)p.D2 & 15) == 0);
    if (p.epi & (kEpiDGelu | kEpiAddAux | kEpiMulAux))
      ok = ok && (p.ldaux % 8 == 0) && (((uintptr_t)p.aux & 15) == 0);
    p.vec_ok = ok ? 1 : 0;
  }
  if (((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return -3;
  p.bn = kPairBN;
  CUtensorMap tmA, tmB;
  int rc;
  if (!p.a_mn)
    rc = make_tmap_bf16_2d(&tmA, A, (uint64_t)p.K, (uint64_t)a_rows, (uint64_t)lda, 64, 128);
  else
    rc = make_tmap_bf16_2d(&tmA, A, (uint64_t)p.M, (uint64_t)a_rows, (uint64_t)lda, 64, 64);
  if (rc) return rc;
  if (!p.b_mn)
    rc = make_tmap_bf16_2d(&tmB, B, (uint64_t)p.K, (uint64_t)b_rows, (uint64_t)ldb, 64, kPairBN / 2);
  else
    rc = make_tmap_bf16_2d(&tmB, B, (uint64_t)p.N, (uint64_t)b_rows, (uint64_t)ldb, 64, 64);
  if (rc) return rc;

  int stages = (200 * 1024) / kPairStageBytes;
  if (stages > kGemmMaxStages) stages = kGemmMaxStages;
  p.stages = stages;
  const int smem_bytes = stages * kPairStageBytes + 1024;
  if (g_pair_max_dyn == 0) {
    cudaFuncAttributes fa;
    cudaError_t e = cudaFuncGetAttributes(&fa, gemm_bf16_pair_kernel);
    if (e != cudaSuccess) return (int)e;
    const int max_dyn = 232448 - (int)fa.sharedSizeBytes;
    e = cudaFuncSetAttribute(gemm_bf16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_dyn);
    if (e != cudaSuccess) return (int)e;
    // how many pairs the device holds at once (a persistent grid must not exceed it)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * sm_count());
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, gemm_bf16_pair_kernel, &cfg);
    if (e != cudaSuccess || n <= 0) { cudaGetLastError(); n = sm_count() / 2; }
    g_pair_clusters = n;
    g_pair_max_dyn = max_dyn;
  }
  if (smem_bytes > g_pair_max_dyn) return -6;
  const int num_m = (p.M + 2 * kGemmBM - 1) / (2 * kGemmBM);
  const int num_n = (p.N + kPairBN - 1) / kPairBN;
  long long tiles = (long long)num_m * num_n;
  if (p.groups_k > 0) tiles *= p.groups_k;
  int pairs = g_pair_clusters;
  if (tiles < pairs) pairs = (int)tiles;
  p.gemm_ctas = 2 * pairs;
  {
    cudaError_t e = launch_pdl(gemm_bf16_pair_kernel, dim3(2 * pairs), dim3(kThreads), (size_t)smem_bytes, stream,
                               tmA, tmB, p);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)cudaGetLastError();
}

}  // namespace mmj

using namespace mmj;

// Number of CTA pairs the device holds at once for the pair kernel (0 before its first launch).
MMJ_API int mmj_gemm_pair_clusters() { return g_pair_clusters; }

// Plain / fused-epilogue GEMM.
//   a_mn = 0: A is [M, K] row-major (lda);  a_mn = 1: A is [K, M] row-major (lda)
//   b_mn = 0: B is [N, K] row-major (ldb);  b_mn = 1: B is [K, N] row-major (ldb)
//   D[M, N] (ldd) = A_op * B_op^T-style contraction over K, then the epilogue flags in `epi`.
MMJ_API int mmj_gemm_bf16(const void* A, long long lda, int a_mn, const void* B, long long ldb,
                          int b_mn, void* D, long long ldd, int M, int N, int K, int epi,
                          const void* bias, const void* aux, long long ldaux, void* D2,
                          long long ldd2, const float* row_scale, int bn, int* status,
                          void* stream) {
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.bn = bn & 0xfff;          // bit 12 of `bn` asks for 256-row tiles
  p.bm2 = (bn >> 12) & 1;
  p.epi = epi;
  p.D = D; p.ldd = ldd;
  p.D2 = D2; p.ldd2 = ldd2;
  p.bias = bias; p.aux = aux; p.ldaux = ldaux;
  p.row_scale = row_scale;
  p.status = status;
  if ((bn >> 13) & 1)  // bit 13 of `bn`: CTA-pair kernel, 256 x 256 tiles
    return launch_gemm_pair(p, A, lda, a_mn ? K : M, B, ldb, b_mn ? K : N, (cudaStream_t)stream);
  return launch_gemm(p, A, lda, a_mn ? K : M, B, ldb, b_mn ? K : N, 0, (cudaStream_t)stream);
}

// Grouped GEMM for MoE experts: rows of A are sorted by expert and every expert's segment
// starts on a 128-row boundary. tile_group[m_tile] names the expert of each row tile;
// num_m_tiles_dev (device int) is the number of row tiles in use. B holds `groups` weight
// matrices stacked along its row dimension, b_group_rows rows each.
MMJ_API int mmj_gemm_bf16_grouped(const void* A, long long lda, const void* B, long long ldb,
                                  int b_mn, int groups, int b_group_rows, void* D, long long ldd,
                                  int M_cap, int N, int K, int epi, const void* aux,
                                  long long ldaux, const float* row_scale, const int* tile_group,
                                  const int* num_m_tiles_dev, int bn, int* status, void* stream) {
  GemmParams p = {};
  p.M = M_cap; p.N = N; p.K = K;
  p.a_mn = 0; p.b_mn = b_mn;
  p.bn = bn;
  p.epi = epi;
  p.D = D; p.ldd = ldd;
  p.aux = aux; p.ldaux = ldaux;
  p.row_scale = row_scale;
  p.status = status;
  p.tile_group = tile_group;
  p.b_group_rows = b_group_rows;
  p.num_m_tiles_dev = num_m_tiles_dev;
  return launch_gemm(p, A, lda, M_cap, B, ldb, (long long)groups * b_group_rows, 0,
                     (cudaStream_t)stream);
}

// All-gather fused into the GEMM. One operand (A when gather_a != 0, else B) is the
// concatenation along rows of `world` equal shards that live on different GPUs.
// `gathered` is the local full-size buffer (the GEMM reads it through TMA); comm CTAs copy
// each peer shard from peer_src[r] into it in `granule_rows`-row pieces (128 for A, bn for B)
// and publish flags[piece] = epoch, which the TMA producer waits on (bounded). peer_ready
// (may be null) is the local signal pad where rank r stores `epoch` once its shard is final.
MMJ_API int mmj_gemm_bf16_allgather(const void* const* peer_src, void* gathered, int gather_a,
                                    const void* other, long long ld_gathered, long long ld_other,
                                    int other_mn, void* D, long long ldd, int M, int N, int K,
                                    int epi, const void* bias, const void* aux, long long ldaux,
                                    void* D2, long long ldd2, int bn, int world, int rank,
                                    long long shard_bytes, long long flat_off_bytes,
                                    int* flags, const int* peer_ready, int epoch, int comm_ctas,
                                    int* status, void* stream) {
  if (world < 1 || world > kMaxPeers) return -5;
  GemmParams p = {};
  p.src_compact = (gather_a >> 1) & 1;   // bit 1 of gather_a: peers keep compact shards
  gather_a &= 1;
  p.M = M; p.N = N; p.K = K;
  p.bn = bn & 0xfff;          // bit 12 of `bn` asks for 256-row tiles
  p.bm2 = (bn >> 12) & 1;
  bn = p.bn;
  p.epi = epi;
  p.D = D; p.ldd = ldd;
  p.D2 = D2; p.ldd2 = ldd2;
  p.bias = bias; p.aux = aux; p.ldaux = ldaux;
  p.status = status;
  p.world = world; p.rank = rank;
  p.ready_flags = flags; p.flags_rw = flags;
  p.peer_ready = peer_ready;
  p.ready_epoch = epoch;
  p.gather_dst = gathered;
  for (int r = 0; r < world; ++r) p.peer_src[r] = peer_src[r];
  const long long rows = gather_a ? M : N;
  const int granule = gather_a ? kGemmBM : bn;
  p.tile_bytes = (long long)granule * ld_gathered * 2;
  p.gather_total_bytes = rows * ld_gathered * 2;
  p.gather_flat_off = flat_off_bytes;
  p.shard_bytes = shard_bytes;
  if (shard_bytes <= 0 || (shard_bytes & 15) || (flat_off_bytes & 15)) return -6;
  // first tile that holds local data (if any) is visited first
  long long first_local = (long long)rank * shard_bytes - flat_off_bytes;
  if (first_local < 0) first_local = 0;
  int rot_tile = 0;
  if (first_local < p.gather_total_bytes) rot_tile = (int)((first_local + p.tile_bytes - 1) / p.tile_bytes);
  const int ntiles_g = (int)((p.gather_total_bytes + p.tile_bytes - 1) / p.tile_bytes);
  if (rot_tile >= ntiles_g) rot_tile = 0;
  if (gather_a) {
    p.flag_mode = 1;
    p.a_mn = 0; p.b_mn = other_mn;
    p.comm_rot = rot_tile;
    p.m_tile_rot = p.bm2 ? rot_tile / 2 : rot_tile;
    return launch_gemm(p, gathered, ld_gathered, M, other, ld_other, other_mn ? K : N, comm_ctas,
                       (cudaStream_t)stream);
  } else {
    p.flag_mode = 2;
    p.a_mn = other_mn; p.b_mn = 0;
    p.comm_rot = rot_tile;
    p.n_tile_rot = rot_tile;
    return launch_gemm(p, other, ld_other, other_mn ? K : M, gathered, ld_gathered, N, comm_ctas,
                       (cudaStream_t)stream);
  }
}

// GEMM whose result is reduce-scattered over rows: rank `rank` computes a partial D[M, N];
// rows [r*M/world, (r+1)*M/world) are stored into rank r's staging buffer peer_stage[r] at
// slot `rank` (slot_stride elements apart). Each owner later sums its `world` slots
// (mmj_reduce_slots_bf16). Rows are visited starting after the local block so that ranks
// write to different owners at the same time.
MMJ_API int mmj_gemm_bf16_reduce_scatter(const void* A, long long lda, const void* B,
                                         long long ldb, int b_mn, void* const* peer_stage,
                                         long long ldd, long long slot_stride, int M, int N, int K,
                                         int bn, int world, int rank, int* status, void* stream) {
  if (world < 1 || world > kMaxPeers) return -5;
  if (M % world) return -6;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.a_mn = 0; p.b_mn = b_mn;
  p.bn = bn & 0xfff;          // bit 12 of `bn` asks for 256-row tiles
  p.bm2 = (bn >> 12) & 1;
  p.epi = kEpiScatterPeers;
  p.ldd = ldd;
  p.status = status;
  p.world = world; p.rank = rank;
  p.rows_per_rank = M / world;
  p.slot_stride = slot_stride;
  for (int r = 0; r < world; ++r) p.peer_D[r] = peer_stage[r];
  p.D = peer_stage[rank];
  const int bm = kGemmBM * (p.bm2 ? 2 : 1);
  const int num_m = (M + bm - 1) / bm;
  p.m_tile_rot = (int)(((long long)(rank + 1) % world) * p.rows_per_rank / bm) % num_m;
  return launch_gemm(p, A, lda, M, B, ldb, b_mn ? K : N, 0, (cudaStream_t)stream);
}

// Grouped-K GEMM for expert weight gradients: for every group g,
//   D[g][M, N] = sum over rows k in [group_k[2g], group_k[2g+1]) of A[k, :M]^T B[k, :N]
// with A: [rows, M] and B: [rows, N] row-major (both MN-major operands; rows outside every range
// are never read, rows inside a range that hold no token must be zero). D is [groups, M, N].
MMJ_API int mmj_gemm_bf16_grouped_k(const void* A, long long lda, const void* B, long long ldb,
                                    void* D, long long ldd, int rows, int M, int N, int groups,
                                    const int* group_k_dev, int out_f32, int accumulate, int bn,
                                    int* status, void* stream) {
  GemmParams p = {};
  p.M = M; p.N = N; p.K = rows;
  p.a_mn = 1; p.b_mn = 1;
  p.bn = bn & 0xfff;          // bit 12 of `bn` asks for 256-row tiles
  p.bm2 = (bn >> 12) & 1;
  p.epi = (out_f32 ? kEpiOutF32 : 0) | (accumulate ? kEpiAccumulate : 0);
  p.D = D; p.ldd = ldd;
  p.status = status;
  p.groups_k = groups;
  p.group_k = group_k_dev;
  if ((bn >> 13) & 1)  // CTA-pair kernel
    return launch_gemm_pair(p, A, lda, rows, B, ldb, rows, (cudaStream_t)stream);
  return launch_gemm(p, A, lda, rows, B, ldb, rows, 0, (cudaStream_t)stream);
}
