// Kernel parameter block shared by the host launcher and the persistent kernels.
#pragma once
#include <stdint.h>
#include "sched.h"

namespace mkb {

// Epilogue applied to the accumulator tile before it is stored.
enum Epilogue : int {
  EPI_NONE = 0,
  // Output tile = silu(first half of the tile's columns) * second half: the GEMM's N is twice the
  // output width and the B rows are laid out [128 gate rows][128 up rows] per 256-wide tile.
  EPI_SWIGLU = 1,
};

struct OpParams {
  Sched sched;
  int K;
  int k_blocks;          // ceil(K / 64)
  int stages;            // operand ring depth
  int b_mn_major;        // 0: B stored [N,K] (K contiguous); 1: B stored [K,N] (N contiguous)
  int n_comm;            // CTAs [0, n_comm) run only the exchange role, the rest run the GEMM
  int item_vecs;         // RS/AR: 16-byte vectors per exchange work item
  int n_items;           // exchange work items of this rank for this launch
  int push_bulk;         // AllGather push: leave each ring step as one TMA bulk store
  int ag_lead_tiles;     // AllGather push pacing: an item may run this many tiles ahead of the
                         // raster group that consumes its rows (0 = unpaced)
  int ag_fanout;         // AllGather push: one item loads a row group once, stores it to all peers
  int ag_cv_log2;        // AllGather push: 0 = an item is 4 full rows of a row-block; otherwise an
                         // item is all rows of a row-block over a K-range of 2^ag_cv_log2 16-byte
                         // vectors, so that consumers start on a row-block as its first range lands
  int ring_slots;        // ring depth (16-byte slots per lane) of the in-CTA exchange warp
  int use_nvls;          // exchange through NVSwitch multicast addresses when available
  int epilogue;          // Epilogue
  int debug_flags;       // timing diagnostics only (results undefined): 1 = exchange workers skip
                         // the data movement but keep the protocol, 2 = RS epilogue stores locally
  uint32_t epoch_arg;    // GEMM+AR: caller-provided epoch; other ops read SW_EPOCH
  uint64_t wait_limit_ns;

  void* C;               // GEMM output of this rank, bf16 row-major
  long long ldc;         // elements
  uint32_t* sync;        // this rank's synchronisation words (nullptr for the plain GEMM)
  uint32_t* status;      // 4 status words: sync + SW_STATUS, or caller-provided, or nullptr
  uint32_t* peer_sync[kMaxWorld];
  // AG: every rank's gathered-A buffer ([W, M/W, K]); RS/AR: every rank's partial C ([M, N]).
  void* peer_data[kMaxWorld];
  // AR: every rank's C_final ([M, N]).  RS: unused (result overwrites the owner's slice of C).
  void* peer_out[kMaxWorld];
  void* mc_data;         // multicast alias of peer_data (or nullptr)
  void* mc_out;          // multicast alias of peer_out (or nullptr)
  // Splitting the tiles of a partial last round along K (plain GEMM, AllGather+GEMM): fp32
  // scratch for the pieces' accumulators (one 128 x block_n slot per CTA), arrival counters
  // (zeroed by the host before the launch), and the largest number of pieces per tile (0 = off).
  float* split_scratch;
  uint32_t* split_counters;
  int split_max_parts;
  // Diagnostics build only: 16 counters per CTA (cycles each role spent waiting); else nullptr.
  unsigned long long* trace;
};

}  // namespace mkb
