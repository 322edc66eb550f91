// Flash-style attention forward and backward on tcgen05 tensor cores (causal or full, MHA and
// GQA, head_dim 64 or 128), with Q/K/V/dO tiles staged by TMA (128-byte swizzle) and every
// matrix product accumulated in tensor memory.
//
// Forward, one CTA per (128 query rows, head, batch):
//   S = Q K^T in TMEM -> softmax warps read one row per thread (no shuffles needed), keep the
//   running max / sum, write P (bf16) into shared memory in the swizzled K-major layout ->
//   O_part = P V in TMEM -> threads fold O_part into a register accumulator.
// Backward, one CTA per (128 key rows, kv head, batch), looping over the query blocks (and,
// for GQA, over the query heads of the group):
//   S^T = K Q^T and dP^T = V dO^T (TMEM) -> threads rebuild P^T = exp(S^T*scale - lse) and
//   dS^T = P^T o (dP^T - delta), write both to shared memory -> dV += P^T dO, dK += dS^T Q
//   (TMEM, accumulated over the whole loop), dQ = dS K (TMEM, then a TMA reduce-add into the
//   fp32 accumulator in global memory).
// The tiles loaded once by TMA serve both as K-major and as MN-major operands: a 128-row tile
// whose rows are 128 swizzled bytes is the canonical layout of either, read with a different
// descriptor.
//
// The reference attention is a forward-only scalar loop that builds one score row at a time
// (legacy/src/momijo/learn/nn/attention.mojo:122-161); softmax is the default normaliser here.
#include "common.cuh"

#include <cstdlib>

namespace mmj {

constexpr int kAttnThreads = 192;     // forward: TMA warp, MMA warp, 4 softmax warps
constexpr int kAttnBwdThreads = 448;  // backward: TMA warp, MMA warp, 8 compute warps, 4 dQ warps
struct TrueTag { static constexpr bool value = true; };
struct FalseTag { static constexpr bool value = false; };
constexpr int kPanelBytes = 128 * 128;  // 128 rows x 64 bf16

struct AttnParams {
  int B, T, Hq, Hkv;
  int q_col0, k_col0, v_col0;  // column of head 0 inside the Q / K / V tensor maps
  float scale;                 // softmax scale (1/sqrt(D))
  int causal;
  // forward outputs
  __nv_bfloat16* O;
  long long ldo;
  float* lse;  // [B, Hq, T]
  // backward
  const float* delta;  // [B, Hq, T]
  float* dQ;           // fp32 accumulator [B*T, ld_dq]
  long long ld_dq;
  __nv_bfloat16* dK;
  __nv_bfloat16* dV;
  long long ld_dk, ld_dv;
  int dk_col0, dv_col0, dq_col0, o_col0;
  int* status;
  long long* trace;  // nullable; kTraceSlots stamps per CTA
};

// K-major operand descriptor for k-step `k` (16 elements each) of a tile made of 64-column panels.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_addr, int k) {
  return make_smem_desc(tile_addr + (uint32_t)(k >> 2) * kPanelBytes + (uint32_t)(k & 3) * 32, 16,
                        1024);
}
// MN-major operand descriptor: rows are the contraction index, 16 rows per k-step.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile_addr, int k) {
  return make_smem_desc(tile_addr + (uint32_t)k * 2048, kPanelBytes, 1024);
}

// Write 32 consecutive columns [col0, col0+32) of row r into a 128 x 128 bf16 tile stored as
// two 64-column panels with the 128-byte swizzle (16-byte chunk index ^= row & 7).
__device__ __forceinline__ void store_chunk_sw128(uint8_t* tile, int r, int col0,
                                                  const float (&v)[32]) {
  uint8_t* rowp = tile + (col0 >> 6) * kPanelBytes + r * 128;
  const int cbase = (col0 & 63) >> 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 q;
    q.x = pack_bf16x2(v[8 * i + 0], v[8 * i + 1]);
    q.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
    q.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
    q.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
    const int phys = (cbase + i) ^ (r & 7);
    *reinterpret_cast<uint4*>(rowp + phys * 16) = q;
  }
}

// TMA reduce-add of a shared-memory box into a global tensor (element type from the map).
// The x coordinate times the element size must be a multiple of 16 bytes; coordinates are
// never negative here.
__device__ __forceinline__ void tma_reduce_add_3d(const void* tmap, const void* smem_src, int c0,
                                                  int c1, int c2) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.bulk_group [%0, {%2, %3, %4}], [%1];"
      :
      : "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_group_read0() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_group0() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// Optional kernel timeline: when a trace buffer is installed, one compute (or softmax) thread and the
// MMA thread of every CTA store clock64() stamps at their stage boundaries (64 slots per CTA).
constexpr int kTraceSlots = 64;
__device__ __forceinline__ void trace_stamp(long long* trace, int cta, int slot) {
  if (trace != nullptr && slot < kTraceSlots) trace[(long long)cta * kTraceSlots + slot] = clock64();
}

// =============================================================================================
// Forward
// =============================================================================================
template <int D>
__global__ void __launch_bounds__(kAttnThreads, (D == 64) ? 2 : 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  constexpr int NP = D / 64;             // 64-column panels per tile
  constexpr int kTile = NP * kPanelBytes;
  constexpr uint32_t kTmemCols = 256;
  constexpr uint32_t kColS = 0, kColO = 128;
  // head_dim 64 keeps a single V stage so that two CTAs fit in one SM's shared memory (the
  // second CTA's softmax then overlaps this CTA's MMAs); head_dim 128 runs one CTA per SM.
  constexpr int VS = (D == 64) ? 1 : 2;

  extern __shared__ uint8_t smem_raw[];
  // (offset arithmetic on the __shared__ symbol, not an integer round trip, so that the compiler
  // keeps the shared address space and emits shared rather than generic loads and stores)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kTile;      // 2 stages
  uint8_t* sV = sK + 2 * kTile;  // VS stages
  // head_dim 128 (one CTA per SM) has room for two P tiles, so the softmax of block j+1 need not
  // wait for P(j) V(j); head_dim 64 keeps one (its second CTA on the SM fills the gap)
  constexpr int PB = (D == 64) ? 1 : 2;
  constexpr int kPTile = 2 * kPanelBytes;
  uint8_t* sP = sV + VS * kTile;  // PB tiles of 128 x 128 bf16

  __shared__ __align__(8) uint64_t q_full, s_full, p_full, o_full;
  __shared__ __align__(8) uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2], p_free[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_qb = (p.T + 127) / 128;
  const int qb = num_qb - 1 - (int)blockIdx.x;  // heaviest (latest) query blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hkv = h / (p.Hq / p.Hkv);
  const int q0 = qb * 128;
  int kv_end = p.causal ? min(p.T, q0 + 128) : p.T;
  const int nkv = (kv_end + 127) / 128;
  const int cta_lin = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
  const bool tracer = (threadIdx.x == 64);
  if (tracer) {
    trace_stamp(p.trace, cta_lin, 0);
    if (p.trace) {
      uint32_t smid;
      asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
      p.trace[(long long)cta_lin * kTraceSlots + 1] = smid;
      p.trace[(long long)cta_lin * kTraceSlots + 7] = nkv;
    }
  }

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    mbar_init(&s_full, 1);
    mbar_init(&p_full, 4);
    mbar_init(&o_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&p_free[s], 1);
    }
    abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  pdl_wait();  // the set-up above read no tensor of the step
  pdl_trigger();
  if (tracer) trace_stamp(p.trace, cta_lin, 2);

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&q_full, kTile);
#pragma unroll
      for (int pn = 0; pn < NP; ++pn)
        tma_load_3d(sQ + pn * kPanelBytes, &tmQ, &q_full, p.q_col0 + h * D + pn * 64, q0, b);
      for (int j = 0; j < nkv; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[s], ph ^ 1, &abort_flag, p.status, kTimeoutEmpty, j)) break;
        mbar_expect_tx(&k_full[s], kTile);
#pragma unroll
        for (int pn = 0; pn < NP; ++pn)
          tma_load_3d(sK + s * kTile + pn * kPanelBytes, &tmK, &k_full[s],
                      p.k_col0 + hkv * D + pn * 64, j * 128, b);
        const int sv = j % VS;
        const uint32_t phv = (j / VS) & 1;
        if (!mbar_wait(&v_empty[sv], phv ^ 1, &abort_flag, p.status, kTimeoutEmpty, 100 + j)) break;
        mbar_expect_tx(&v_full[sv], kTile);
#pragma unroll
        for (int pn = 0; pn < NP; ++pn)
          tma_load_3d(sV + sv * kTile + pn * kPanelBytes, &tmV, &v_full[sv],
                      p.v_col0 + hkv * D + pn * 64, j * 128, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);
      const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP);
      bool ok = mbar_wait(&q_full, 0, &abort_flag, p.status, kTimeoutFull, -1);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[s], ph, &abort_flag, p.status, kTimeoutFull, j)) return false;
        tc_fence_after();
        const uint32_t aK = smem_u32(sK + s * kTile);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16_ss(tmem_base + kColS, desc_kmajor(aQ, k), desc_kmajor(aK, k), idesc_s,
                       k > 0 ? 1u : 0u);
        umma_commit(&k_empty[s]);
        umma_commit(&s_full);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < nkv && ok; ++j) {
        const int sv = j % VS;
        const uint32_t phv = (j / VS) & 1;
        if (!mbar_wait(&p_full, j & 1, &abort_flag, p.status, kTimeoutFlag, j)) break;
        trace_stamp(p.trace, cta_lin, 8 + j * 6 + 3);
        // P(j) written means S(j) has been consumed: the next score tile goes first, so that
        // the softmax of block j+1 can start while P(j) V(j) is still running
        if (j + 1 < nkv) ok = issue_s(j + 1);
        if (!ok) break;
        if (!mbar_wait(&v_full[sv], phv, &abort_flag, p.status, kTimeoutFull, 100 + j)) break;
        tc_fence_after();
        const uint32_t aV = smem_u32(sV + sv * kTile);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16_ss(tmem_base + kColO, desc_kmajor(aP + (uint32_t)((j % PB) * kPTile), k), desc_mnmajor(aV, k), idesc_o,
                       (j > 0 || k > 0) ? 1u : 0u);
        umma_commit(&v_empty[sv]);
        umma_commit(&p_free[j % PB]);  // this P tile may be overwritten
        umma_commit(&o_full);
      }
    }
  } else {
    // ---------------- softmax / output warps: one query row per thread ----------------
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int q_idx = q0 + row;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
    const float c = p.scale * 1.4426950408889634f;
    // The output accumulator stays in tensor memory (P V accumulates into it); it is rescaled
    // in place only when the running row maximum grows by more than kTau (in the exp2 domain),
    // so most iterations neither read nor write it. Probabilities are then bounded by 2^kTau,
    // which bf16 / fp32 hold comfortably, and the final 1/l normalisation makes the result exact.
    constexpr float kTau = 8.0f;
    float m_used = -1.0e30f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nkv; ++j) {
      if (!mbar_wait_warp(&s_full, j & 1, &abort_flag, p.status, kTimeoutTmemFull, j)) { ok = false; break; }
      tc_fence_after();
      if (tracer) trace_stamp(p.trace, cta_lin, 8 + j * 6 + 0);
      const int kv0 = j * 128;
      const bool need_mask = (p.causal && (kv0 + 127 > q0)) || (kv0 + 128 > p.T);
      uint32_t s[128];
      tmem_ld_32x32(t_lane + kColS + 0, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_ld_32x32(t_lane + kColS + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
      tmem_ld_32x32(t_lane + kColS + 64, *reinterpret_cast<uint32_t(*)[32]>(&s[64]));
      tmem_ld_32x32(t_lane + kColS + 96, *reinterpret_cast<uint32_t(*)[32]>(&s[96]));
      tmem_ld_wait();
      if (tracer) trace_stamp(p.trace, cta_lin, 8 + j * 6 + 1);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          const int kv = kv0 + i;
          if (kv >= p.T || (p.causal && kv > q_idx)) s[i] = 0xff800000u;  // -inf
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 128; i += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(s[i + 0]));
        mx1 = fmaxf(mx1, __uint_as_float(s[i + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(s[i + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(s[i + 3]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      const bool grow = (mx - m_used) * c > kTau;  // false for fully masked rows (mx = -inf)
      if (__any_sync(0xffffffffu, grow ? 1 : 0)) {
        float alpha = 1.0f;
        if (grow) {
          alpha = exp2f((m_used - mx) * c);
          l *= alpha;
          m_used = mx;
        }
        if (j > 0) {
          // P(j-1) V(j-1) must have landed before the accumulator is rescaled
          if (!mbar_wait_warp(&o_full, (j - 1) & 1, &abort_flag, p.status, kTimeoutTmemFull, 100 + j)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int cc = 0; cc < D / 32; ++cc) {
            uint32_t r[32];
            tmem_ld_32x32(t_lane + kColO + cc * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32(t_lane + kColO + cc * 32, r);
          }
          tmem_st_wait();
        }
      }
      // P(j-1) V(j-1) reads the P tile that is about to be overwritten: it must have finished. (It
      // was issued after S(j) and takes a fraction of the time spent above, so this wait is normally
      // already satisfied; without it the order would only be a matter of timing.)
      // (one barrier per P tile: each sees one completion per use of its tile, so a wait for the
      // previous use can never be overtaken by a later phase)
      if (j >= PB) {
        if (!mbar_wait_warp(&p_free[j % PB], ((j / PB) - 1) & 1, &abort_flag, p.status, kTimeoutTmemFull, 200 + j)) { ok = false; break; }
      }
      const float mc = m_used * c;
      float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        float(&pv)[32] = *reinterpret_cast<float(*)[32]>(&s[cc * 32]);  // exponentiate in place
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          pv[i + 0] = exp2f(fmaf(pv[i + 0], c, -mc));
          pv[i + 1] = exp2f(fmaf(pv[i + 1], c, -mc));
          pv[i + 2] = exp2f(fmaf(pv[i + 2], c, -mc));
          pv[i + 3] = exp2f(fmaf(pv[i + 3], c, -mc));
          sum0 += pv[i + 0]; sum1 += pv[i + 1]; sum2 += pv[i + 2]; sum3 += pv[i + 3];
        }
        store_chunk_sw128(sP + (j % PB) * kPTile, row, cc * 32, pv);
      }
      l += (sum0 + sum1) + (sum2 + sum3);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full);
      if (tracer) trace_stamp(p.trace, cta_lin, 8 + j * 6 + 2);
    }
    if (tracer) trace_stamp(p.trace, cta_lin, 4);
    // final: wait for the last P V, normalise and store
    if (ok && nkv > 0)
      ok = mbar_wait_warp(&o_full, (nkv - 1) & 1, &abort_flag, p.status, kTimeoutTmemFull, 999);
    if (ok) {
      tc_fence_after();
      const float inv = (l > 0.f) ? 1.0f / l : 0.f;
      __nv_bfloat16* dst = p.O + ((long long)b * p.T + q_idx) * p.ldo + p.o_col0 + h * D;
#pragma unroll
      for (int cc = 0; cc < D / 32; ++cc) {
        uint32_t r[32];
        tmem_ld_32x32(t_lane + kColO + cc * 32, r);
        tmem_ld_wait();
        if (q_idx < p.T) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 q;
            q.x = pack_bf16x2(__uint_as_float(r[8 * i + 0]) * inv, __uint_as_float(r[8 * i + 1]) * inv);
            q.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv);
            q.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv);
            q.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv);
            reinterpret_cast<uint4*>(dst + cc * 32)[i] = q;
          }
        }
      }
      if (q_idx < p.T && p.lse != nullptr)
        p.lse[((long long)b * p.Hq + h) * p.T + q_idx] =
            (l > 0.f) ? (m_used * p.scale + __logf(l)) : -INFINITY;
    }
  }

  if (tracer) trace_stamp(p.trace, cta_lin, 5);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (tracer) trace_stamp(p.trace, cta_lin, 6);
}

// =============================================================================================
// Forward, two query tiles per CTA, 64-key blocks, double-buffered score tiles (the default)
// =============================================================================================
// One persistent CTA per SM walks a list of work items, heaviest first; an item is 256 query rows (two
// 128-row tiles) of one (batch, head). Three warpgroups: warps 0..3 = TMA producer (warp 0), one MMA issuer
// per query tile (warps 1 and 2; warp 1 owns the TMEM allocation) and an idle warp; warps 4..7 = softmax
// group of tile 0; warps 8..11 = softmax group of tile 1 (one query row per thread). A softmax group reads
// its score tile from tensor memory, writes the probabilities back over the first columns of the same tile
// as packed bf16 pairs, and the P V product takes them from there as its tensor-memory A operand: P never
// touches shared memory. Three things keep the tensor core out of the groups' dependency chain:
//   * each query tile has its own MMA-issuing thread (warps 1 and 2);
//   * a key block is 64 keys and every query tile owns TWO score buffers in tensor memory
//     (S_t[0], S_t[1], 64 columns each): the MMA thread issues S_t(j+1) before the group has finished
//     block j, so a group that has stored P_t(j) finds S_t(j+1) waiting and starts on it at once;
//     per key block the MMA thread does  [wait P_t(j)]  P_t(j) V_j -> O_t,  Q_t K_(j+2)^T -> S_t[j & 1];
//   * probabilities are rounded to bf16 with integer arithmetic (add half an ulp, take the upper
//     halves with one byte permute) instead of the conversion instruction, which shares the
//     transcendental pipe with the exponentials.
// Tensor memory: S0[0] S0[1] S1[0] S1[1] | O0 | O1 = 256 + 2 D columns; P_t(j) overwrites the first 32
// columns of S_t[j & 1] (64 probabilities as bf16 pairs). Every P_t(j) V_j commits to o_done[t][j & 1];
// a group waits on it only before it rescales O_t (rare: the running maximum must have grown by more
// than 2^8) and before the final normalisation.
__device__ __forceinline__ uint32_t pack_bf16x2_halfup(float lo, float hi) {
  // lo, hi >= 0 (probabilities): adding 0x8000 to the bit pattern rounds the upper 16 bits half-up
  const uint32_t a = __float_as_uint(lo) + 0x8000u, b = __float_as_uint(hi) + 0x8000u;
  return __byte_perm(a, b, 0x7632);
}

template <int D>
__global__ void __launch_bounds__(384, 1)
attn_fwd3_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  constexpr int NP = D / 64;
  constexpr int kQTile = NP * kPanelBytes;         // 128 query rows
  constexpr int kKVPanel = 64 * 128;               // 64 key rows x 64 bf16
  constexpr int kKVTile = NP * kKVPanel;           // 64 key rows x D
  constexpr int KS = (D == 64) ? 6 : 4;            // K and V stages
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColO = 256;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sQ = smem;                   // 2 tiles
  uint8_t* sK = sQ + 2 * kQTile;        // KS stages
  uint8_t* sV = sK + KS * kKVTile;      // KS stages

  __shared__ __align__(8) uint64_t q_full[2], q_empty[2], o_free[2];
  __shared__ __align__(8) uint64_t s_full[2][2], p_full[2][2], o_done[2][2];
  __shared__ __align__(8) uint64_t k_full[KS], k_empty[KS], v_full[KS], v_empty[KS];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqp = (p.T + 255) / 256;
  const int nbh = p.B * p.Hq;
  const int n_items = nqp * nbh;
  const int group = p.Hq / p.Hkv;

  if (threadIdx.x == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(&q_full[t], 1);
      mbar_init(&q_empty[t], 1);
      mbar_init(&o_free[t], 4);
      for (int b = 0; b < 2; ++b) {
        mbar_init(&s_full[t][b], 1);
        mbar_init(&p_full[t][b], 4);
        mbar_init(&o_done[t][b], 1);
      }
    }
    for (int s = 0; s < KS; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 2);   // one arrival per query tile (its MMA thread)
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 2);
    }
    abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  pdl_wait();  // the set-up above touched no global memory
  pdl_trigger();

  auto decode = [&](int w, int& qp, int& h, int& b) {
    qp = nqp - 1 - w / nbh;  // later (longer) query pairs first
    const int bh = w % nbh;
    h = bh % p.Hq;
    b = bh / p.Hq;
  };
  // 64-key blocks of tile t of query pair qp (0 when the tile lies beyond T)
  auto blocks_of = [&](int qp, int t) -> int {
    const int q0 = qp * 256 + t * 128;
    if (q0 >= p.T) return 0;
    const int kv_end = p.causal ? min(p.T, q0 + 128) : p.T;
    return (kv_end + 63) / 64;
  };

  if (warp == 0) {
    // ======================= TMA producer =======================
    if (lane == 0) {
      uint32_t qn[2] = {0, 0};
      uint32_t kc = 0;  // ring position of this item's block 0 (K and V rings advance together per item)
      bool ok = true;
      for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
        int qp, h, b;
        decode(w, qp, h, b);
        const int hkv = h / group;
        const int nb[2] = {blocks_of(qp, 0), blocks_of(qp, 1)};
        const int n1 = max(nb[0], nb[1]);
        for (int t = 0; t < 2 && ok; ++t) {
          if (nb[t] == 0) continue;
          if (!mbar_wait(&q_empty[t], (qn[t] & 1) ^ 1, &abort_flag, p.status, kTimeoutEmpty, 300 + t)) { ok = false; break; }
          ++qn[t];
          mbar_expect_tx(&q_full[t], kQTile);
#pragma unroll
          for (int pn = 0; pn < NP; ++pn)
            tma_load_3d(sQ + t * kQTile + pn * kPanelBytes, &tmQ, &q_full[t], p.q_col0 + h * D + pn * 64,
                        qp * 256 + t * 128, b);
        }
        auto load_k = [&](int j) -> bool {
          const uint32_t c = kc + (uint32_t)j;
          const int s = c % KS;
          if (!mbar_wait(&k_empty[s], ((c / KS) & 1) ^ 1, &abort_flag, p.status, kTimeoutEmpty, j)) return false;
          mbar_expect_tx(&k_full[s], kKVTile);
#pragma unroll
          for (int pn = 0; pn < NP; ++pn)
            tma_load_3d(sK + s * kKVTile + pn * kKVPanel, &tmK, &k_full[s], p.k_col0 + hkv * D + pn * 64, j * 64, b);
          return true;
        };
        auto load_v = [&](int j) -> bool {
          const uint32_t c = kc + (uint32_t)j;
          const int s = c % KS;
          if (!mbar_wait(&v_empty[s], ((c / KS) & 1) ^ 1, &abort_flag, p.status, kTimeoutEmpty, 100 + j)) return false;
          mbar_expect_tx(&v_full[s], kKVTile);
#pragma unroll
          for (int pn = 0; pn < NP; ++pn)
            tma_load_3d(sV + s * kKVTile + pn * kKVPanel, &tmV, &v_full[s], p.v_col0 + hkv * D + pn * 64, j * 64, b);
          return true;
        };
        // the order the MMA thread consumes them in: K0 K1 V0 K2 V1 K3 ...
        for (int j = 0; j < n1 && ok; ++j) {
          ok = load_k(j);
          if (ok && j >= 1) ok = load_v(j - 1);
        }
        if (ok && n1 > 0) ok = load_v(n1 - 1);
        kc += (uint32_t)n1;
      }
    }
  } else if (warp == 1 || warp == 2) {
    // ======================= MMA issuers: warp 1 drives query tile 0, warp 2 tile 1 =======================
    // (a single issuing thread spends about 1400 cycles per tile and key block on waits, descriptors,
    // MMAs and commits; with one thread per tile the two tiles' chains no longer queue behind each other)
    if (lane == 0) {
      const int t = warp - 1;
      const uint32_t idesc_s = make_idesc_bf16(128, 64, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);
      uint32_t qn = 0;
      uint32_t pc[2] = {0, 0};  // P tiles consumed so far, per buffer
      uint32_t on = 0;
      uint32_t kc = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
        int qp, h, b;
        decode(w, qp, h, b);
        const int nbt = blocks_of(qp, t);
        const int n1 = max(blocks_of(qp, 0), blocks_of(qp, 1));
        // S_t(j) = Q_t K_j^T into buffer j & 1
        auto issue_s = [&](int j) -> bool {
          const uint32_t c = kc + (uint32_t)j;
          const int s = c % KS;
          if (!mbar_wait(&k_full[s], (c / KS) & 1, &abort_flag, p.status, kTimeoutFull, j)) return false;
          tc_fence_after();
          const uint32_t aQ = smem_u32(sQ + t * kQTile), aK = smem_u32(sK + s * kKVTile);
          const uint32_t d = tmem_base + (uint32_t)(t * 128 + (j & 1) * 64);
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            // K tile: 64 rows, 64-column panels of 8 KiB
            const uint64_t dk = make_smem_desc(aK + (uint32_t)(k >> 2) * kKVPanel + (uint32_t)(k & 3) * 32, 16, 1024);
            umma_bf16_ss(d, desc_kmajor(aQ, k), dk, idesc_s, k > 0 ? 1u : 0u);
          }
          umma_commit(&k_empty[s]);   // this tile's share of the K block's release
          if (j + 1 == nbt) umma_commit(&q_empty[t]);
          umma_commit(&s_full[t][j & 1]);
          return true;
        };
        if (nbt > 0) {
          if (!mbar_wait(&q_full[t], qn & 1, &abort_flag, p.status, kTimeoutFull, 400 + t)) { ok = false; break; }
          ++qn;
          ok = issue_s(0);
          if (ok && nbt > 1) ok = issue_s(1);
        }
        for (int j = 0; j < n1 && ok; ++j) {
          const uint32_t c = kc + (uint32_t)j;
          const int sv = c % KS;
          if (j >= nbt) {
            // a key block only the other tile reads: hand in this tile's share of its release, but only
            // once the block has been loaded (an earlier arrival would count for the stage's previous block)
            if (!mbar_wait(&k_full[sv], (c / KS) & 1, &abort_flag, p.status, kTimeoutFull, 800 + j)) { ok = false; break; }
            mbar_arrive(&k_empty[sv]);
            if (!mbar_wait(&v_full[sv], (c / KS) & 1, &abort_flag, p.status, kTimeoutFull, 900 + j)) { ok = false; break; }
            mbar_arrive(&v_empty[sv]);
            continue;
          }
          const int bf = j & 1;
          if (!mbar_wait(&p_full[t][bf], pc[bf] & 1, &abort_flag, p.status, kTimeoutFlag, 500 + j)) { ok = false; break; }
          ++pc[bf];
          if (j == 0 && on > 0) {
            if (!mbar_wait(&o_free[t], (on - 1) & 1, &abort_flag, p.status, kTimeoutTmemEmpty, 600 + t)) { ok = false; break; }
          }
          if (!mbar_wait(&v_full[sv], (c / KS) & 1, &abort_flag, p.status, kTimeoutFull, 100 + j)) { ok = false; break; }
          tc_fence_after();
          const uint32_t aV = smem_u32(sV + sv * kKVTile);
          const uint32_t aP = tmem_base + (uint32_t)(t * 128 + bf * 64);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // V tile as an MN-major B operand: 16 key rows per step, 64-wide panels 8 KiB apart
            const uint64_t dv = make_smem_desc(aV + (uint32_t)k * 2048, kKVPanel, 1024);
            umma_bf16_ts(tmem_base + kColO + t * D, aP + k * 8, dv, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&v_empty[sv]);
          umma_commit(&o_done[t][bf]);   // P_t(j) V_j has landed in O_t
          if (j + 1 == nbt) ++on;
          if (j + 2 < nbt) ok = issue_s(j + 2);
        }
        kc += (uint32_t)n1;
      }
    }
  } else if (warp >= 4) {
    // ======================= softmax groups: one query row per thread =======================
    const int t = (warp - 4) >> 2;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t colO = kColO + t * D;
    const float c = p.scale * 1.4426950408889634f;
    constexpr float kTau = 8.0f;
    uint32_t sn[2] = {0, 0};   // score tiles consumed so far, per buffer
    uint32_t pn[2] = {0, 0};   // P tiles produced so far, per buffer (= P V products expected)
    bool ok = true;
    const bool tracer = (p.trace != nullptr) && (lane == 0) && (quad == 0) && (t == 0);
    for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
      int qp, h, b;
      decode(w, qp, h, b);
      const int nkv = blocks_of(qp, t);
      if (nkv == 0) continue;
      const int q0 = qp * 256 + t * 128;
      const int q_idx = q0 + row;
      const bool tr = tracer && (w == (int)blockIdx.x);
      if (tr && t == 0) {
        p.trace[(long long)blockIdx.x * kTraceSlots + 7] = nkv;
        trace_stamp(p.trace, blockIdx.x, 0);
      }
      float m_used = -1.0e30f, l = 0.f;
      for (int j = 0; j < nkv; ++j) {
        const int bf = j & 1;
        const uint32_t colS = (uint32_t)(t * 128 + bf * 64);
        if (!mbar_wait_warp(&s_full[t][bf], sn[bf] & 1, &abort_flag, p.status, kTimeoutTmemFull, j)) { ok = false; break; }
        ++sn[bf];
        tc_fence_after();
        if (tr && j < 6) trace_stamp(p.trace, blockIdx.x, 8 + 24 * t + 4 * j + 0);
        const int kv0 = j * 64;
        const bool need_mask = (p.causal && (kv0 + 63 > q0)) || (kv0 + 64 > p.T);
        uint32_t s[64];
        tmem_ld_32x32(t_lane + colS + 0, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
        tmem_ld_32x32(t_lane + colS + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
        tmem_ld_wait();
        if (tr && j < 6) trace_stamp(p.trace, blockIdx.x, 8 + 24 * t + 4 * j + 1);
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const int kv = kv0 + i;
            if (kv >= p.T || (p.causal && kv > q_idx)) s[i] = 0xff800000u;  // -inf
          }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
          mx0 = fmaxf(mx0, __uint_as_float(s[i + 0]));
          mx1 = fmaxf(mx1, __uint_as_float(s[i + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(s[i + 2]));
          mx3 = fmaxf(mx3, __uint_as_float(s[i + 3]));
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        if (tr && j < 6) trace_stamp(p.trace, blockIdx.x, 8 + 24 * t + 4 * j + 2);
        const bool grow = (mx - m_used) * c > kTau;  // false for fully masked rows (mx = -inf)
        if (__any_sync(0xffffffffu, grow ? 1 : 0)) {
          float alpha = 1.0f;
          if (grow) {
            alpha = exp2f((m_used - mx) * c);
            l *= alpha;
            m_used = mx;
          }
          if (j > 0) {
            // O_t holds the blocks up to j - 1 once P_t(j-1) V has landed (its commit is the newest on
            // the other buffer's barrier; never more than one completion away, so the parity is safe)
            const int ob = bf ^ 1;
            if (!mbar_wait_warp(&o_done[t][ob], (pn[ob] - 1) & 1, &abort_flag, p.status, kTimeoutTmemFull, 700 + j)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int cc = 0; cc < D / 32; ++cc) {
              uint32_t r[32];
              tmem_ld_32x32(t_lane + colO + cc * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st_32x32(t_lane + colO + cc * 32, r);
            }
          }
        }
        const float mc = m_used * c;
        float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
        // 64 probabilities as bf16 pairs, packed in place: pair m lands in s[m], which the loop has
        // already consumed (it reads s[2m ...], never behind its writes)
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float e0 = exp2f(fmaf(__uint_as_float(s[2 * i + 0]), c, -mc));
          const float e1 = exp2f(fmaf(__uint_as_float(s[2 * i + 1]), c, -mc));
          const float e2 = exp2f(fmaf(__uint_as_float(s[2 * i + 2]), c, -mc));
          const float e3 = exp2f(fmaf(__uint_as_float(s[2 * i + 3]), c, -mc));
          sum0 += e0; sum1 += e1; sum2 += e2; sum3 += e3;
          s[i + 0] = pack_bf16x2_halfup(e0, e1);
          s[i + 1] = pack_bf16x2_halfup(e2, e3);
        }
        tmem_st_32x32(t_lane + colS, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
        l += (sum0 + sum1) + (sum2 + sum3);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[t][bf]);
        ++pn[bf];
        if (tr && j < 6) trace_stamp(p.trace, blockIdx.x, 8 + 24 * t + 4 * j + 3);
      }
      if (!ok) break;
      if (tr) trace_stamp(p.trace, blockIdx.x, 2 + 2 * t);
      // final: wait for the last P V of this tile, normalise and store
      {
        const int lb = (nkv - 1) & 1;
        if (!mbar_wait_warp(&o_done[t][lb], (pn[lb] - 1) & 1, &abort_flag, p.status, kTimeoutTmemFull, 999)) { ok = false; break; }
      }
      tc_fence_after();
      const float inv = (l > 0.f) ? 1.0f / l : 0.f;
      __nv_bfloat16* dst = p.O + ((long long)b * p.T + q_idx) * p.ldo + p.o_col0 + h * D;
#pragma unroll
      for (int cc = 0; cc < D / 32; ++cc) {
        uint32_t r[32];
        tmem_ld_32x32(t_lane + colO + cc * 32, r);
        tmem_ld_wait();
        if (cc == D / 32 - 1) {
          // the accumulator is in registers: the next item may overwrite O_t
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&o_free[t]);
        }
        if (q_idx < p.T) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 q;
            q.x = pack_bf16x2(__uint_as_float(r[8 * i + 0]) * inv, __uint_as_float(r[8 * i + 1]) * inv);
            q.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv);
            q.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv);
            q.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv);
            reinterpret_cast<uint4*>(dst + cc * 32)[i] = q;
          }
        }
      }
      if (q_idx < p.T && p.lse != nullptr)
        p.lse[((long long)b * p.Hq + h) * p.T + q_idx] = (l > 0.f) ? (m_used * p.scale + __logf(l)) : -INFINITY;
      if (tr) trace_stamp(p.trace, blockIdx.x, 3 + 2 * t);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// =============================================================================================
// Backward
// =============================================================================================
// delta[b, h, t] = sum_d dO[b, t, h, d] * O[b, t, h, d]; D/8 lanes per (row, head), 16 bytes per
// lane and tensor, so a warp covers 4 (head_dim 64) or 2 (head_dim 128) heads of a row at once.
// The same lanes clear the fp32 dQ accumulator (8 values each) that the backward kernel adds into.
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ O, long long ldo, int o_col0,
                                  const __nv_bfloat16* __restrict__ dO, long long lddo, int do_col0,
                                  float* __restrict__ delta, float* __restrict__ dq_zero, long long ld_dq,
                                  int dq_col0, int B, int T, int H, int D) {
  pdl_wait();
  pdl_trigger();
  const int lp = D >> 3;  // lanes per item: 8 or 16
  const long long gt = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long item = gt / lp;
  const int sub = (int)(gt - item * lp);
  const long long total = (long long)B * T * H;
  const bool live = item < total;
  float s = 0.f;
  int h = 0;
  long long bt = 0;
  if (live) {
    h = (int)(item % H);
    bt = item / H;
    const uint4 a = *reinterpret_cast<const uint4*>(O + bt * ldo + o_col0 + h * D + sub * 8);
    const uint4 c = *reinterpret_cast<const uint4*>(dO + bt * lddo + do_col0 + h * D + sub * 8);
    if (dq_zero != nullptr) {
      float4* z = reinterpret_cast<float4*>(dq_zero + bt * ld_dq + dq_col0 + h * D + sub * 8);
      z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
      z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const uint32_t av[4] = {a.x, a.y, a.z, a.w}, cv[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = unpack_bf16x2(av[i]), y = unpack_bf16x2(cv[i]);
      s = fmaf(x.x, y.x, fmaf(x.y, y.y, s));
    }
  }
  for (int o = lp >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (live && sub == 0) {
    const long long b = bt / T, t = bt - b * T;
    delta[(b * H + h) * T + t] = s;
  }
}

struct BwdCtl {
  uint64_t kv_full, s_full, p_full, pds_free, acc_full, stat_full;
  uint64_t dq_full[2], dq_read[2];
  uint64_t dq_staged, stage_free;
  uint64_t qdo_full[4], qdo_empty[4];
  float s_lse[2][128], s_delta[2][128];
  uint32_t tmem_slot;
  int abort_flag;
};

// Backward kernel. Warp roles (14 warps): 0 = TMA producer, 1 = MMA issuer and TMEM owner,
// 2..9 = compute (P^T and dS^T from S^T and dP^T, then the dK/dV epilogue), 10..13 = dQ drain
// (TMEM -> registers -> swizzled fp32 staging tile -> TMA reduce-add into global; per-thread
// red.global.add would spend one L1 sector slot per 16 bytes and starve the compute warps' own
// shared-memory traffic). A warp reaches the 32 TMEM lanes of its quadrant (warp
// index mod 4) only, so two compute warps share each quadrant and split the columns; two
// compute warps per scheduler also hide each other's dependent-issue and TMEM-load latency.
template <int D>
__global__ void __launch_bounds__(kAttnBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const __grid_constant__ CUtensorMap tmdQ, const AttnParams p) {
  constexpr int NP = D / 64;
  constexpr int kTile = NP * kPanelBytes;
  // head_dim 64: three Q/dO stages, so that a stage released by the MMAs of block i is refilled
  // (about 1.5 us of TMA latency) before block i+2 needs it, and two dQ accumulators.
  // head_dim 128 has shared memory for one stage and TMEM columns for one dQ that aliases S^T.
  constexpr int kStages = (D == 64) ? 3 : 1;
  constexpr bool kAliasdQ = (D == 128);
  constexpr int kDQB = kAliasdQ ? 1 : 2;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColSt = 0, kColdPt = 128, kColdV = 256, kColdK = 256 + D;
  constexpr uint32_t kColdQ = kAliasdQ ? 0u : (256u + 2u * D);  // + D per extra buffer
  constexpr int kPdsBytes = 2 * kPanelBytes;                    // one 128 x 128 bf16 tile

  extern __shared__ uint8_t smem_raw[];
  // (offset arithmetic on the __shared__ symbol, not an integer round trip, so that the compiler
  // keeps the shared address space and emits shared rather than generic loads and stores)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sK = smem;
  uint8_t* sV = sK + kTile;
  uint8_t* sQ = sV + kTile;              // kStages
  uint8_t* sdO = sQ + kStages * kTile;   // kStages
  uint8_t* sPt = sdO + kStages * kTile;  // 128 x 128 bf16
  uint8_t* sdSt = sPt + kPdsBytes;       // 128 x 128 bf16
  uint8_t* sDQ = sdSt + kPdsBytes;       // 128 x 64 fp32: two 32-column panels, 128-byte swizzle

  // Barriers and the lse / delta staging live behind the tiles in dynamic shared memory: with
  // head_dim 64 the tiles alone take 224 KB, and a static segment in front of them would push
  // the 1024-byte alignment padding over the per-CTA limit.
  BwdCtl& ctl = *reinterpret_cast<BwdCtl*>(sDQ + 2 * kPanelBytes);
  {
    uint32_t dyn_bytes;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    const uint32_t need = (uint32_t)(reinterpret_cast<uint8_t*>(&ctl) - smem_raw) + sizeof(BwdCtl);
    if (need > dyn_bytes) {  // uniform over the CTA: nothing allocated yet, just leave
      if (threadIdx.x == 0) report(p.status, kBadArgument, (int)need);
      return;
    }
  }
  uint64_t &kv_full = ctl.kv_full, &s_full = ctl.s_full, &p_full = ctl.p_full;
  uint64_t &pds_free = ctl.pds_free, &acc_full = ctl.acc_full, &stat_full = ctl.stat_full;
  uint64_t *dq_full = ctl.dq_full, *dq_read = ctl.dq_read;
  uint64_t &dq_staged = ctl.dq_staged, &stage_free = ctl.stage_free;
  uint64_t *qdo_full = ctl.qdo_full, *qdo_empty = ctl.qdo_empty;
  float(*s_lse)[128] = ctl.s_lse;
  float(*s_delta)[128] = ctl.s_delta;
  uint32_t& tmem_slot = ctl.tmem_slot;
  int& abort_flag = ctl.abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // One-dimensional grid ordered by work: with a causal mask key block 0 meets every query block and
  // the last key block only one, so all CTAs of key block 0 are dispatched first, then those of key
  // block 1 and so on (longest first; the tail of the grid is made of the one-block CTAs).
  const int n_heads_b = p.Hkv * p.B;
  const int jb = (int)blockIdx.x / n_heads_b;  // key block
  const int hb = (int)blockIdx.x - jb * n_heads_b;
  const int hkv = hb % p.Hkv, b = hb / p.Hkv;
  const int group = p.Hq / p.Hkv;
  const int num_qb = (p.T + 127) / 128;
  const int kv0 = jb * 128;
  const int i_begin = p.causal ? jb : 0;
  const int n_i = num_qb - i_begin;   // query blocks per head
  const int n_iter = n_i * group;     // (query head in group) x (query block)
  const int cta_lin = (int)blockIdx.x;
  const bool tracer = (threadIdx.x == 64);
  if (tracer) {
    trace_stamp(p.trace, cta_lin, 0);
    if (p.trace) {
      uint32_t smid;
      asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
      p.trace[(long long)cta_lin * kTraceSlots + 1] = smid;
      p.trace[(long long)cta_lin * kTraceSlots + 7] = n_iter;
    }
  }

  if (threadIdx.x == 0) {
    mbar_init(&kv_full, 1);
    mbar_init(&s_full, 1);
    mbar_init(&p_full, 8);
    mbar_init(&pds_free, 1);
    mbar_init(&acc_full, 1);
    mbar_init(&stat_full, 128);
    mbar_init(&dq_staged, 4);
    mbar_init(&stage_free, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&dq_full[s], 1);
      mbar_init(&dq_read[s], 4);
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmdO);
    prefetch_tmap(&tmdQ);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  pdl_wait();  // the set-up above read no tensor of the step
  pdl_trigger();
  if (tracer) trace_stamp(p.trace, cta_lin, 2);

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&kv_full, 2 * kTile);
#pragma unroll
      for (int pn = 0; pn < NP; ++pn) {
        tma_load_3d(sK + pn * kPanelBytes, &tmK, &kv_full, p.k_col0 + hkv * D + pn * 64, kv0, b);
        tma_load_3d(sV + pn * kPanelBytes, &tmV, &kv_full, p.v_col0 + hkv * D + pn * 64, kv0, b);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        const int hq = hkv * group + it / n_i;
        const int qi = i_begin + it % n_i;
        if (!mbar_wait(&qdo_empty[s], ph ^ 1, &abort_flag, p.status, kTimeoutEmpty, it)) break;
        mbar_expect_tx(&qdo_full[s], 2 * kTile);
#pragma unroll
        for (int pn = 0; pn < NP; ++pn) {
          tma_load_3d(sQ + s * kTile + pn * kPanelBytes, &tmQ, &qdo_full[s],
                      p.q_col0 + hq * D + pn * 64, qi * 128, b);
          tma_load_3d(sdO + s * kTile + pn * kPanelBytes, &tmdO, &qdo_full[s],
                      p.o_col0 + hq * D + pn * 64, qi * 128, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_st = make_idesc_bf16(128, 128, 0, 0);  // K/V (K-major) x Q/dO (K-major)
      const uint32_t idesc_dkv = make_idesc_bf16(128, D, 0, 1);   // P^T/dS^T (K-major) x dO/Q (MN)
      const uint32_t idesc_dq = make_idesc_bf16(128, D, 1, 1);    // dS^T as MN-major A x K (MN)
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV);
      const uint32_t aPt = smem_u32(sPt), adSt = smem_u32(sdSt);
      bool ok = mbar_wait(&kv_full, 0, &abort_flag, p.status, kTimeoutFull, -1);
      trace_stamp(p.trace, cta_lin, 3);
      // S^T = K Q^T and dP^T = V dO^T of block `it` (the Q/dO stage must have landed)
      auto issue_scores = [&](int it) -> bool {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        if (!mbar_wait(&qdo_full[s], ph, &abort_flag, p.status, kTimeoutFull, it)) return false;
        tc_fence_after();
        const uint32_t aQ = smem_u32(sQ + s * kTile), adO = smem_u32(sdO + s * kTile);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16_ss(tmem_base + kColSt, desc_kmajor(aK, k), desc_kmajor(aQ, k), idesc_st,
                       k > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16_ss(tmem_base + kColdPt, desc_kmajor(aV, k), desc_kmajor(adO, k), idesc_st,
                       k > 0 ? 1u : 0u);
        umma_commit(&s_full);
        return true;
      };
      if (ok && n_iter > 0) ok = issue_scores(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it % kStages;
        const int qb = it % kDQB;
        if (!mbar_wait(&p_full, it & 1, &abort_flag, p.status, kTimeoutFlag, it)) { ok = false; break; }
        tc_fence_after();
        trace_stamp(p.trace, cta_lin, 8 + it * 6 + 5);
        // S^T / dP^T of this block are consumed. With a dQ accumulator of its own the next
        // block's scores can go first (its exponentials then overlap the MMAs below), provided
        // its Q/dO stage has landed; otherwise they follow the gradient MMAs.
        bool scores_issued = (it + 1 >= n_iter);
        if (!kAliasdQ && !scores_issued) {
          const int s1 = (it + 1) % kStages;
          if (mbar_try_wait(&qdo_full[s1], ((it + 1) / kStages) & 1)) {
            ok = issue_scores(it + 1);
            scores_issued = true;
          }
        }
        const uint32_t aQ = smem_u32(sQ + s * kTile), adO = smem_u32(sdO + s * kTile);
        // dV += P^T dO ; dK += dS^T Q   (contraction over the 128 query rows)
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16_ss(tmem_base + kColdV, desc_kmajor(aPt, k), desc_mnmajor(adO, k), idesc_dkv,
                       (it > 0 || k > 0) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16_ss(tmem_base + kColdK, desc_kmajor(adSt, k), desc_mnmajor(aQ, k), idesc_dkv,
                       (it > 0 || k > 0) ? 1u : 0u);
        // dQ = dS K  (contraction over the 128 key rows; dS^T tile read as an MN-major A)
        if (!kAliasdQ && it >= kDQB) {
          if (!mbar_wait(&dq_read[qb], ((it / kDQB) - 1) & 1, &abort_flag, p.status, kTimeoutFlag, 200 + it)) { ok = false; break; }
          tc_fence_after();
        }
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16_ss(tmem_base + kColdQ + qb * D, desc_mnmajor(adSt, k), desc_mnmajor(aK, k),
                       idesc_dq, k > 0 ? 1u : 0u);
        umma_commit(&qdo_empty[s]);
        umma_commit(&pds_free);
        umma_commit(&dq_full[qb]);
        if (it + 1 == n_iter) umma_commit(&acc_full);
        if (!scores_issued) {
          if (kAliasdQ) {
            // dQ shares the S^T columns: the next scores wait until dQ has been drained
            if (!mbar_wait(&dq_read[0], it & 1, &abort_flag, p.status, kTimeoutFlag, 300 + it)) { ok = false; break; }
            tc_fence_after();
          }
          ok = issue_scores(it + 1);
        }
      }
    }
  } else if (warp < 10) {
    // ---------------- compute warps: one key row and half of the columns per thread --------
    const int quad = warp & 3;
    const int chalf = (warp - 2) >> 2;  // which half of the columns this warp handles
    const int row = quad * 32 + lane;   // key row inside the block
    const int kv_idx = kv0 + row;
    const int ctid = threadIdx.x - 64;  // 0..255; the first 128 also stage lse / delta
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
    const float c = p.scale * 1.4426950408889634f;
    const float l2e = 1.4426950408889634f;
    bool ok = true;

    // lse / delta of query block `it` go to shared memory one iteration ahead: the global loads
    // are issued at the top of iteration it-1 and stored at its end, so the wait on stat_full
    // at the top of iteration `it` normally finds the phase complete.
    float st_l = 0.f, st_d = 0.f;
    auto stat_load = [&](int it) {
      if (ctid < 128 && it < n_iter) {
        const int hq = hkv * group + it / n_i;
        const int q = (i_begin + it % n_i) * 128 + ctid;
        const long long off = ((long long)b * p.Hq + hq) * p.T + q;
        st_l = (q < p.T) ? p.lse[off] * l2e : 0.f;
        st_d = (q < p.T) ? p.delta[off] : 0.f;
      }
    };
    auto stat_store = [&](int it) {
      if (ctid < 128 && it < n_iter) {
        s_lse[it & 1][ctid] = st_l;
        s_delta[it & 1][ctid] = st_d;
        mbar_arrive(&stat_full);
      }
    };
    stat_load(0);
    stat_store(0);

    for (int it = 0; it < n_iter; ++it) {
      const int qbase = (i_begin + it % n_i) * 128;
      const float* lse_s = s_lse[it & 1];
      const float* delta_s = s_delta[it & 1];
      stat_load(it + 1);
      if (!mbar_wait_warp(&stat_full, it & 1, &abort_flag, p.status, kTimeoutFlag, 500 + it)) { ok = false; break; }
      if (!mbar_wait_warp(&s_full, it & 1, &abort_flag, p.status, kTimeoutTmemFull, it)) { ok = false; break; }
      tc_fence_after();
      if (tracer) trace_stamp(p.trace, cta_lin, 8 + it * 6 + 0);
      const bool need_mask = (p.causal && (qbase < kv0 + 127)) || (qbase + 128 > p.T) ||
                             (kv0 + 128 > p.T);
      // Both variants are straight-line code (the mask is a select, not a branch), so that the
      // 32 independent exp / multiply chains of a chunk interleave.
      auto chunk = [&](auto masked_tag, int cc, float (&pt)[32], float (&ds)[32]) {
        constexpr bool kMasked = decltype(masked_tag)::value;
        const int col0 = chalf * 64 + cc * 32;
        uint32_t rs[32], rp[32];
        tmem_ld_32x32(t_lane + kColSt + col0, rs);
        tmem_ld_32x32(t_lane + kColdPt + col0, rp);
        tmem_ld_wait();
#pragma unroll
        for (int i4 = 0; i4 < 8; ++i4) {
          const float4 l4 = *reinterpret_cast<const float4*>(&lse_s[col0 + 4 * i4]);
          const float4 d4 = *reinterpret_cast<const float4*>(&delta_s[col0 + 4 * i4]);
          const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
          const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int i = 4 * i4 + u;
            float e = exp2f(fmaf(__uint_as_float(rs[i]), c, -ls[u]));
            if (kMasked) {
              const int q = qbase + col0 + i;
              const bool dead = (q >= p.T) | (kv_idx >= p.T) | ((p.causal != 0) & (kv_idx > q));
              e = dead ? 0.f : e;
            }
            pt[i] = e;
            ds[i] = e * (__uint_as_float(rp[i]) - dl[u]);
          }
        }
      };
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        float pt[32], ds[32];
        if (need_mask) chunk(TrueTag{}, cc, pt, ds);
        else chunk(FalseTag{}, cc, pt, ds);
        if (tracer && cc == 0) trace_stamp(p.trace, cta_lin, 8 + it * 6 + 1);
        if (cc == 0 && it > 0) {
          // the gradient MMAs of the previous block read P^T / dS^T: they must have finished
          if (!mbar_wait_warp(&pds_free, (it - 1) & 1, &abort_flag, p.status, kTimeoutFlag, 600 + it)) { ok = false; break; }
        }
        store_chunk_sw128(sPt, row, chalf * 64 + cc * 32, pt);
        store_chunk_sw128(sdSt, row, chalf * 64 + cc * 32, ds);
      }
      if (!ok) break;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full);
      if (tracer) trace_stamp(p.trace, cta_lin, 8 + it * 6 + 2);
      if (ctid < 128 && it + 1 < n_iter) {
        // Every compute warp has passed its wait on stat_full(it) once p_full(it) completes;
        // arriving for the next phase any earlier could complete it before a slow warp looked
        // at this one. The scores of block it+1 need p_full(it) as well, so this costs nothing.
        if (!mbar_wait_warp(&p_full, it & 1, &abort_flag, p.status, kTimeoutFlag, 800 + it)) { ok = false; break; }
        stat_store(it + 1);
      }
    }
    // all MMAs into dV / dK have completed once acc_full fires
    if (ok && n_iter > 0)
      ok = mbar_wait_warp(&acc_full, 0, &abort_flag, p.status, kTimeoutTmemFull, 700);
    tc_fence_after();
    // tcgen05.ld is warp-collective: the condition around it must be warp-uniform; only the
    // global stores are predicated per row.
    const bool warp_ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
    const bool row_ok = kv_idx < p.T;
    if (tracer) trace_stamp(p.trace, cta_lin, 4);
    if (warp_ok && n_iter > 0) {
      __nv_bfloat16* dk = p.dK + ((long long)b * p.T + kv_idx) * p.ld_dk + p.dk_col0 + hkv * D;
      __nv_bfloat16* dv = p.dV + ((long long)b * p.T + kv_idx) * p.ld_dv + p.dv_col0 + hkv * D;
#pragma unroll
      for (int c2 = 0; c2 < D / 64; ++c2) {
        const int cc = chalf * (D / 64) + c2;
        uint32_t r[32];
        tmem_ld_32x32(t_lane + kColdV + cc * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 q;
          q.x = pack_bf16x2(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]));
          q.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
          q.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
          q.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
          if (row_ok) reinterpret_cast<uint4*>(dv + cc * 32)[i] = q;
        }
        tmem_ld_32x32(t_lane + kColdK + cc * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 q;
          q.x = pack_bf16x2(__uint_as_float(r[8 * i + 0]) * p.scale, __uint_as_float(r[8 * i + 1]) * p.scale);
          q.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * p.scale, __uint_as_float(r[8 * i + 3]) * p.scale);
          q.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * p.scale, __uint_as_float(r[8 * i + 5]) * p.scale);
          q.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * p.scale, __uint_as_float(r[8 * i + 7]) * p.scale);
          if (row_ok) reinterpret_cast<uint4*>(dk + cc * 32)[i] = q;
        }
      }
    } else if (warp_ok && row_ok && n_iter == 0) {
      // no query block attends to this key block: gradients are zero
      __nv_bfloat16* dk = p.dK + ((long long)b * p.T + kv_idx) * p.ld_dk + p.dk_col0 + hkv * D;
      __nv_bfloat16* dv = p.dV + ((long long)b * p.T + kv_idx) * p.ld_dv + p.dv_col0 + hkv * D;
      for (int i = chalf * (D / 16); i < (chalf + 1) * (D / 16); ++i) {
        reinterpret_cast<uint4*>(dk)[i] = make_uint4(0, 0, 0, 0);
        reinterpret_cast<uint4*>(dv)[i] = make_uint4(0, 0, 0, 0);
      }
    }
  } else {
    // ---------------- dQ drain warps: one query row per thread ----------------
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
    const bool elected = (threadIdx.x == 320);  // issues the TMA reductions; also the tracer
    uint8_t* my_row = sDQ + row * 128;
    int u = 0;  // staging-tile uses so far (D / 64 per query block)
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int qb = it % kDQB;
      if (!mbar_wait_warp(&dq_full[qb], (it / kDQB) & 1, &abort_flag, p.status, kTimeoutTmemFull, 100 + it)) break;
      tc_fence_after();
      if (elected) trace_stamp(p.trace, cta_lin, 8 + it * 6 + 3);
      const int hq = hkv * group + it / n_i;
      const int q0 = (i_begin + it % n_i) * 128;
#pragma unroll
      for (int h2 = 0; h2 < D / 64; ++h2, ++u) {
        uint32_t r[2][32];
        tmem_ld_32x32(t_lane + kColdQ + qb * D + h2 * 64, r[0]);
        tmem_ld_32x32(t_lane + kColdQ + qb * D + h2 * 64 + 32, r[1]);
        tmem_ld_wait();
        if (h2 == D / 64 - 1) {
          // the accumulator is in registers: hand its TMEM columns back right away
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&dq_read[qb]);
        }
        // the previous reduction must have finished reading the staging tile
        if (u > 0 && !mbar_wait_warp(&stage_free, (u - 1) & 1, &abort_flag, p.status, kTimeoutFlag, 900 + it)) { ok = false; break; }
#pragma unroll
        for (int pn = 0; pn < 2; ++pn) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 v;
            v.x = __uint_as_float(r[pn][4 * j + 0]) * p.scale;
            v.y = __uint_as_float(r[pn][4 * j + 1]) * p.scale;
            v.z = __uint_as_float(r[pn][4 * j + 2]) * p.scale;
            v.w = __uint_as_float(r[pn][4 * j + 3]) * p.scale;
            *reinterpret_cast<float4*>(my_row + pn * kPanelBytes + ((j ^ (row & 7)) << 4)) = v;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&dq_staged);
        if (elected) {
          if (!mbar_wait(&dq_staged, u & 1, &abort_flag, p.status, kTimeoutFlag, 1000 + it)) { ok = false; }
          else {
            // rows past T are clipped by the tensor map (3-D: columns, rows of one batch, batch)
#pragma unroll
            for (int pn = 0; pn < 2; ++pn)
              tma_reduce_add_3d(&tmdQ, sDQ + pn * kPanelBytes,
                                p.dq_col0 + hq * D + h2 * 64 + pn * 32, q0, b);
            bulk_commit_group();
            bulk_wait_group_read0();
            mbar_arrive(&stage_free);
          }
        }
        ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
        if (!ok) break;
      }
      if (elected) trace_stamp(p.trace, cta_lin, 8 + it * 6 + 4);
    }
    if (elected) bulk_wait_group0();  // reductions in flight finish before the CTA retires
  }

  if (tracer) trace_stamp(p.trace, cta_lin, 5);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (tracer) trace_stamp(p.trace, cta_lin, 6);
}

static long long* g_attn_trace = nullptr;
static long long g_attn_trace_ctas = 0;

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

void ensure_context();  // gemm_sm100.cu

static EncodeTiledFn attn_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(f);
  }
  return fn;
}

// [B, T, cols] bf16 view with row stride ld: dims {cols, T, B}, box {64, 128, 1}.
static int make_tmap_btc(CUtensorMap* out, const void* base, int B, int T, long long cols,
                         long long ld, int box_rows = 128) {
  EncodeTiledFn fn = attn_encode_fn();
  if (fn == nullptr) return -1;
  ensure_context();
  if (ld % 8 || ((uintptr_t)base & 15)) return -2;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)T, (cuuint64_t)B};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)ld * 2 * (cuuint64_t)T};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return (r == CUDA_SUCCESS) ? 0 : (int)r;
}

// fp32 accumulator [B*T, ld] viewed as [B][T][ld]; boxes of 32 columns x 128 rows, 128-byte swizzle
static int make_tmap_f32_btc(CUtensorMap* out, const void* base, int B, int T, long long ld) {
  EncodeTiledFn fn = attn_encode_fn();
  if (fn == nullptr) return -1;
  ensure_context();
  if (ld % 4 || ((uintptr_t)base & 15)) return -2;
  cuuint64_t dims[3] = {(cuuint64_t)ld, (cuuint64_t)T, (cuuint64_t)B};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 4, (cuuint64_t)ld * 4 * (cuuint64_t)T};
  cuuint32_t box[3] = {32, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return (r == CUDA_SUCCESS) ? 0 : (int)r;
}

}  // namespace mmj

using namespace mmj;

// q/k/v: [B*T, ld*] bf16 matrices in which head h of Q starts at column q_col0 + h*D (same for
// K/V with Hkv heads). O: [B*T, ldo] with head h at o_col0 + h*D. lse: [B, Hq, T] fp32.
MMJ_API int mmj_attn_fwd(const void* q, long long ldq, int q_col0, const void* k, long long ldk,
                         int k_col0, const void* v, long long ldv, int v_col0, void* O,
                         long long ldo, int o_col0, float* lse, int B, int T, int Hq, int Hkv,
                         int D, float scale, int causal, int* status, void* stream) {
  if (D != 64 && D != 128) return -10;
  if (Hkv <= 0 || Hq % Hkv) return -11;
  if (ldo % 8 || o_col0 % 8) return -12;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_tmap_btc(&tq, q, B, T, ldq, ldq))) return rc;
  if ((rc = make_tmap_btc(&tk, k, B, T, ldk, ldk))) return rc;
  if ((rc = make_tmap_btc(&tv, v, B, T, ldv, ldv))) return rc;
  AttnParams p = {};
  p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
  p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0;
  p.scale = scale; p.causal = causal;
  p.O = (__nv_bfloat16*)O; p.ldo = ldo; p.o_col0 = o_col0;
  p.lse = lse;
  p.status = status;
  // Default (3): persistent kernel, two query tiles per CTA, 64-key blocks with double-buffered score
  // tiles. MOMIJO_ATTN_FWD=1 selects the older one-tile-per-CTA kernel (kept for comparison).
  static int fwd_mode = -1;
  if (fwd_mode < 0) {
    const char* e = getenv("MOMIJO_ATTN_FWD");
    fwd_mode = e ? atoi(e) : 3;
  }
  if (fwd_mode == 3) {
    static bool b64 = false, b128 = false;
    static int sms3 = 0;
    if (sms3 == 0) {
      int dev = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms3, cudaDevAttrMultiProcessorCount, dev);
    }
    CUtensorMap tk64, tv64;
    if ((rc = make_tmap_btc(&tk64, k, B, T, ldk, ldk, 64))) return rc;
    if ((rc = make_tmap_btc(&tv64, v, B, T, ldv, ldv, 64))) return rc;
    const long long n_items = (long long)((T + 255) / 256) * Hq * B;
    const unsigned g = (unsigned)(n_items < sms3 ? n_items : sms3);
    p.trace = (g_attn_trace && (long long)g <= g_attn_trace_ctas) ? g_attn_trace : nullptr;
    if (D == 64) {
      const int smem = 2 * kPanelBytes + 2 * 6 * 8192 + 1024;
      if (!b64) {
        cudaFuncSetAttribute(attn_fwd3_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        b64 = true;
      }
      launch_pdl(attn_fwd3_kernel<64>, dim3(g), dim3(384), (size_t)smem, (cudaStream_t)stream, tq, tk64, tv64,
                 p);
    } else {
      const int smem = 2 * 2 * kPanelBytes + 2 * 4 * 16384 + 1024;
      if (!b128) {
        cudaFuncSetAttribute(attn_fwd3_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        b128 = true;
      }
      launch_pdl(attn_fwd3_kernel<128>, dim3(g), dim3(384), (size_t)smem, (cudaStream_t)stream, tq, tk64, tv64,
                 p);
    }
    return (int)cudaGetLastError();
  }
  dim3 grid((T + 127) / 128, Hq, B);
  p.trace = (g_attn_trace && (long long)grid.x * grid.y * grid.z <= g_attn_trace_ctas) ? g_attn_trace : nullptr;
  static bool attr64 = false, attr128 = false;
  if (D == 64) {
    const int smem = 4 * kPanelBytes + 2 * kPanelBytes + 1024;  // Q + 2 K + 1 V + P
    if (!attr64) {
      cudaFuncSetAttribute(attn_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      attr64 = true;
    }
    attn_fwd_kernel<64><<<grid, kAttnThreads, smem, (cudaStream_t)stream>>>(tq, tk, tv, p);
  } else {
    const int smem = 5 * 2 * kPanelBytes + 2 * 2 * kPanelBytes + 1024;  // Q + 2 K + 2 V + 2 P
    if (!attr128) {
      cudaFuncSetAttribute(attn_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      attr128 = true;
    }
    attn_fwd_kernel<128><<<grid, kAttnThreads, smem, (cudaStream_t)stream>>>(tq, tk, tv, p);
  }
  return (int)cudaGetLastError();
}

// Install (or clear, with nullptr) the timeline buffer of the attention kernels: int64
// [ctas * 64], written by whichever of them is launched next. Launches whose grid has more CTAs than `ctas` leave it untouched.
MMJ_API int mmj_attn_set_trace(void* buf, long long ctas) {
  g_attn_trace = reinterpret_cast<long long*>(buf);
  g_attn_trace_ctas = buf ? ctas : 0;
  return 0;
}

// dQ_accum: fp32 [B*T, ld_dq]; its Hq*D columns from dq_col0 are cleared by the delta kernel, then the
// backward kernel adds into them.
// delta: fp32 scratch [B, Hq, T] (filled here). dK/dV: bf16 outputs.
MMJ_API int mmj_attn_bwd(const void* q, long long ldq, int q_col0, const void* k, long long ldk,
                         int k_col0, const void* v, long long ldv, int v_col0, const void* O,
                         long long ldo, int o_col0, const void* dO, long long lddo, int do_col0,
                         const float* lse, float* delta, float* dQ_accum, long long ld_dq,
                         int dq_col0, void* dK, long long ld_dk, int dk_col0, void* dV,
                         long long ld_dv, int dv_col0, int B, int T, int Hq, int Hkv, int D,
                         float scale, int causal, int* status, void* stream) {
  if (D != 64 && D != 128) return -10;
  if (Hkv <= 0 || Hq % Hkv) return -11;
  if (ld_dk % 8 || ld_dv % 8 || dk_col0 % 8 || dv_col0 % 8 || ld_dq % 4 || dq_col0 % 4) return -12;
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_tmap_btc(&tq, q, B, T, ldq, ldq))) return rc;
  if ((rc = make_tmap_btc(&tk, k, B, T, ldk, ldk))) return rc;
  if ((rc = make_tmap_btc(&tv, v, B, T, ldv, ldv))) return rc;
  if ((rc = make_tmap_btc(&tdo, dO, B, T, lddo, lddo))) return rc;
  CUtensorMap tdq;
  if (dq_col0 % 4) return -13;
  if ((rc = make_tmap_f32_btc(&tdq, dQ_accum, B, T, ld_dq))) return rc;
  {
    if (((uintptr_t)O & 15) || (ldo & 7) || (o_col0 & 7) || (do_col0 & 7)) return -1;
    const long long lanes = (long long)B * T * Hq * (D / 8);
    const int threads = 256;
    const long long blocks = (lanes + threads - 1) / threads;
    launch_pdl(attn_delta_kernel, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream,
               (const __nv_bfloat16*)O, ldo, o_col0, (const __nv_bfloat16*)dO, lddo, do_col0, delta,
               (((uintptr_t)dQ_accum & 15) == 0) ? dQ_accum : (float*)nullptr, ld_dq, dq_col0, B, T, Hq, D);
  }
  AttnParams p = {};
  p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
  p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0;
  p.o_col0 = do_col0;  // the dO map is addressed with o_col0 inside the kernel
  p.scale = scale; p.causal = causal;
  p.lse = const_cast<float*>(lse);
  p.delta = delta;
  p.dQ = dQ_accum; p.ld_dq = ld_dq; p.dq_col0 = dq_col0;
  p.dK = (__nv_bfloat16*)dK; p.ld_dk = ld_dk; p.dk_col0 = dk_col0;
  p.dV = (__nv_bfloat16*)dV; p.ld_dv = ld_dv; p.dv_col0 = dv_col0;
  p.status = status;
  p.trace = g_attn_trace;
  dim3 grid((unsigned)(((T + 127) / 128) * Hkv * B));
  if (g_attn_trace && (long long)grid.x > g_attn_trace_ctas) p.trace = nullptr;
  static bool attr64 = false, attr128 = false;
  if (D == 64) {
    // K,V + 3x(Q,dO) + P^T,dS^T + dQ staging = 224 KB of tiles; the control block and the alignment
    // padding take what is left of the 227 KB a CTA may have (the kernel checks that they fit)
    const int smem = 232448;
    if (!attr64) {
      cudaFuncSetAttribute(attn_bwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      attr64 = true;
    }
    launch_pdl(attn_bwd_kernel<64>, grid, dim3(kAttnBwdThreads), (size_t)smem, (cudaStream_t)stream, tq, tk, tv,
               tdo, tdq, p);
  } else {
    const int smem = 232448;  // 224 KB of tiles as well: K,V + Q,dO + P^T,dS^T + dQ staging
    if (!attr128) {
      cudaFuncSetAttribute(attn_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      attr128 = true;
    }
    launch_pdl(attn_bwd_kernel<128>, grid, dim3(kAttnBwdThreads), (size_t)smem, (cudaStream_t)stream, tq, tk, tv,
               tdo, tdq, p);
  }
  return (int)cudaGetLastError();
}
