// Parameter block shared by the tcgen05 GEMM kernel and its host launchers.
#pragma once
#include <stdint.h>

namespace mmj {

constexpr int kGemmBM = 128;
constexpr int kGemmBK = 64;
constexpr int kGemmMaxStages = 8;
constexpr int kMaxPeers = 8;

// Epilogue flag bits.
enum GemmEpi : int {
  kEpiBias = 1,        // + bias[col] (bf16)
  kEpiGelu = 2,        // store pre-activation to D2, then GELU(tanh)
  kEpiDGelu = 4,       // * gelu'(aux[row, col])
  kEpiAddAux = 8,      // + aux[row, col] (residual)
  kEpiOutF32 = 16,     // D is fp32 (else bf16)
  kEpiAccumulate = 32, // D += result (read-modify-write)
  kEpiSilu = 64,       // v = silu(v)  (no pre-activation kept)
  kEpiMulAux = 128,    // v *= aux[row, col]
  kEpiScatterPeers = 256,  // rows of D go to the rank that owns them (GEMM -> reduce-scatter)
  kEpiRowScale = 512,  // v *= row_scale[row] (fp32), e.g. router weights in MoE combine
};

struct GemmParams {
  int M, N, K;
  int a_mn, b_mn;  // 0: operand is K-major ([rows, K]); 1: MN-major ([K, rows])
  int bn;          // N tile: 64, 128 or 256
  int bm2;         // 1: tiles are 256 rows tall (two 128-row MMAs share every B stage)
  int comm_rot;    // first gather granule the communication CTAs visit (granule units)
  int stages;
  int epi;
  int vec_ok;  // epilogue may use 16-byte vector accesses
  void* D;
  long long ldd;
  void* D2;
  long long ldd2;
  const void* bias;
  const void* aux;
  long long ldaux;
  const float* row_scale;
  int* status;

  // Grouped GEMM (MoE experts). tile_group[m_tile] gives the group of each 128-row tile;
  // B rows (K-major) or B k-rows (MN-major) of group g start at g * b_group_rows.
  const int* tile_group;
  int b_group_rows;
  // Number of valid 128-row tiles lives on the device (expert counts are only known there).
  const int* num_m_tiles_dev;
  // Grouped-K mode: groups_k > 0 selects per-group contraction ranges group_k[2g], group_k[2g+1]
  // (device array); the output of group g starts at row g * M.
  const int* group_k;
  int groups_k;

  // Gathered operand (all-gather fused into the GEMM): a tile may only be loaded once
  // ready_flags[tile] >= ready_epoch. flag_mode 0: off, 1: per 128-row tile of A,
  // 2: per bn-row tile of B.
  const int* ready_flags;
  int flag_mode;
  int ready_epoch;
  // Tile order rotation so that each rank starts on the rows it already has.
  int m_tile_rot;
  int n_tile_rot;

  // In-kernel all-gather: CTAs with blockIdx.x >= gemm_ctas copy peer shards into the
  // local gathered buffer and publish ready_flags.
  int gemm_ctas;
  int world, rank;
  const void* peer_src[kMaxPeers];  // peer_src[r]: base of rank r's shard (peer pointer)
  void* gather_dst;                 // local full buffer
  // The gathered operand is a window [gather_flat_off, gather_flat_off + gather_total_bytes)
  // of a flat symmetric buffer that is sharded in equal pieces of shard_bytes per rank: the
  // byte at flat offset o is owned by rank o / shard_bytes. peer_src[r] points at the start of
  // the window in rank r's memory.
  // src_compact: every rank keeps only its own shard, and peer_src[r] points at the start of rank
  // r's shard (not at the window): the byte at flat offset o is read from
  // peer_src[o / shard_bytes] + o % shard_bytes, and the local rank's piece is copied as well.
  int src_compact;
  long long shard_bytes;
  long long gather_flat_off;
  long long gather_total_bytes;
  long long tile_bytes;             // bytes per flag granule (128 rows of A or bn rows of B)
  int* flags_rw;                    // same array as ready_flags, writable
  const int* peer_ready;            // local signal pad: peer_ready[r] >= ready_epoch => shard r final

  // GEMM -> reduce-scatter: rows [r*rows_per_rank, (r+1)*rows_per_rank) of the result are
  // stored into peer_D[r] at slot `rank` (partial sums, reduced by the owner afterwards).
  void* peer_D[kMaxPeers];
  int rows_per_rank;
  long long slot_stride;  // elements between slots in the owner's staging buffer
};

}  // namespace mmj
