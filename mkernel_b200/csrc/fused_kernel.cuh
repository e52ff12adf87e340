// One persistent sm_100a kernel for the tensor-parallel GEMM + collective operators.
//
// Roles inside a compute CTA (256 threads):
//   warp 0      TMA producer: fills a shared-memory ring of (A 128x64, B block_n x 64) stages.
//   warp 1      one thread issues tcgen05.mma into one of two TMEM accumulators.
//   warp 2      tile publisher (RS/AR): after a tile is in memory, fence and raise its flag on
//               every owner.
//   warp 3      exchange worker: pulls exchange work items from a per-rank queue while the GEMM
//               runs (see below).  Its loads/stores use the LSU, which the MMA pipeline does not.
//   warps 4-7   epilogue: tcgen05.ld -> bf16 -> transpose through shared memory -> 128-byte row
//               segments to global memory (local, or the owner GPU for ReduceScatter).
// CTAs [0, n_comm) are dedicated exchange CTAs: all 8 warps are exchange workers (used when the
// GEMM cannot fill the machine anyway, e.g. the decode-shaped AllReduce).
//
// Exchange work items (handed out in order by an atomic counter, so early items meet early data):
//   AllGather      push one 4-row group of the own A shard into a peer's gathered buffer with
//                  posted remote stores (or into all peers with one NVSwitch multicast store),
//                  then fence and raise the group's flag on the receiver.
//   ReduceScatter  GEMM tiles were stored straight into the owner's buffer (slab = producing
//                  rank); an item sums one chunk of the W local slabs (fp32, fixed rank order)
//                  in place once the row-block's flags are all up.
//   AllReduce      partials stay with their producer; an item fetches one chunk from all W ranks,
//                  sums it and stores the result into every rank's output.
// A worker keeps 12-20 KB of reads in flight in a private shared-memory ring filled by cp.async.
//
// Every wait is bounded: when a wait expires the CTA records {code, where, detail} in the status
// words, raises an abort flag that all other waits observe, and the kernel drains and returns.
//
// Behaviour follows the reference operators (semantics only): AllGather+GEMM
// src/ag_gemm_warp_specialized.cu:166-580, GEMM+ReduceScatter src/gemm_rs_blackwell.cu:374-615,
// GEMM+AllReduce src/gemm_ar_blackwell.cu:57-610.
#pragma once
#include "op_params.h"
#include "ptx.cuh"

namespace mkb {

// Timing diagnostics (skipping loads, MMAs or data movement; per-role wait counters) exist only
// in builds made with -DMKB_DIAG; the default build compiles every such branch away.
#ifdef MKB_DIAG
constexpr bool kDiag = true;
#else
constexpr bool kDiag = false;
#endif
__device__ __forceinline__ bool diag(const OpParams& p, int bit) {
  return kDiag && (p.debug_flags & bit) != 0;
}
// Cycle counter read used only by the diagnostics build.
__device__ __forceinline__ long long diag_clock(bool on) { return on ? clock64() : 0ll; }

// Barrier slots inside the CTA's barrier block (8 bytes each).
enum BarSlot : int {
  BAR_FULL = 0,      // [0,8)   operand stage filled by TMA           (compute CTAs)
  BAR_EMPTY = 8,     // [8,16)  operand stage consumed by the MMAs
  BAR_TFULL = 16,    // [16,18) accumulator ready for the epilogue
  BAR_TEMPTY = 18,   // [18,20) accumulator drained
  BAR_STORED = 20,   // [20,22) tile written to global memory by all four epilogue warps
  BAR_COUNT = 32,
};

struct WaitCtx {
  uint32_t* status;            // global status words (may be null)
  volatile uint32_t* s_abort;  // CTA-wide abort flag in shared memory
  uint64_t limit_ns;
  uint32_t where;              // (blockIdx << 8) | role
};

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __noinline__ void report_failure(const WaitCtx& c, int code, uint32_t d0, uint32_t d1) {
  if (c.status != nullptr) {
    if (atomicCAS(c.status, 0u, static_cast<uint32_t>(code)) == 0u) {
      c.status[1] = c.where;
      c.status[2] = d0;
      c.status[3] = d1;
      __threadfence();
    }
  }
  *c.s_abort = 1u;
}

template <bool kSleep, class Pred>
__device__ __noinline__ bool slow_wait(const WaitCtx& c, Pred pred, int code, uint32_t d0,
                                       uint32_t d1) {
  uint32_t it = 0;
  uint64_t t0 = 0;
  while (true) {
    if (pred()) return true;
    ++it;
    if (kSleep && it > 16) __nanosleep(it > 2048 ? 400 : 40);
    if ((it & 127u) == 0u) {
      if (*c.s_abort != 0u) return false;
      if (c.status != nullptr && ptx::ld_relaxed_sys(c.status) != 0u) {
        *c.s_abort = 1u;
        return false;
      }
      const uint64_t now = global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > c.limit_ns) {
        report_failure(c, code, d0, d1);
        return false;
      }
    }
  }
}

// Returns false when the wait expired or another role aborted.
template <bool kSleep, class Pred>
__device__ __forceinline__ bool bounded_wait(const WaitCtx& c, Pred pred, int code, uint32_t d0,
                                             uint32_t d1) {
  if (pred()) return true;
  return slow_wait<kSleep>(c, pred, code, d0, d1);
}

// "This rank has entered (or left) launch e" slots only move forward: a peer that is already one
// launch ahead has certainly passed launch `epoch` (wrap-safe comparison).
__device__ __forceinline__ bool reached(uint32_t flag, uint32_t epoch) {
  return static_cast<int32_t>(flag - epoch) >= 0;
}

__device__ __forceinline__ bool wait_mbar(const WaitCtx& c, uint32_t bar, uint32_t parity,
                                          uint32_t d0) {
  return bounded_wait<false>(c, [&] { return ptx::mbar_try_wait(bar, parity); },
                             ST_TIMEOUT_PIPE, d0, parity);
}

// Timing diagnostics (debug_flags & 4): low 32 bits of %globaltimer at a few protocol events,
// written to the otherwise unused sync words [24, 32).
__device__ __forceinline__ void stamp(const OpParams& p, int slot) {
  if (diag(p, 4) && p.sync != nullptr)
    p.sync[24 + slot] = static_cast<uint32_t>(global_timer_ns());
}

// Same, keeping the latest time over all callers (the event's last occurrence in the launch).
__device__ __forceinline__ void stamp_max(const OpParams& p, int slot) {
  if (diag(p, 4) && p.sync != nullptr)
    atomicMax(p.sync + 24 + slot, static_cast<uint32_t>(global_timer_ns()));
}

// The split plan and the per-CTA work list live in sched.h (host + device, unit-tested on the
// host); these wrappers bind them to the kernel's parameter block.
template <int CG>
__device__ __forceinline__ SplitPlan make_split(const OpParams& p, int total_tiles, int n_comp) {
  if (p.split_scratch == nullptr) return plan_split(total_tiles, n_comp, CG, p.k_blocks, 0);
  return plan_split(total_tiles, n_comp, CG, p.k_blocks, p.split_max_parts);
}
template <int CG>
__device__ __forceinline__ bool work_item(const OpParams& p, const SplitPlan& sp, int total_tiles,
                                          int n_comp, int cta, int it, WorkItem& w) {
  return cta_work_item(sp, total_tiles, n_comp, CG, p.k_blocks, cta, it, &w);
}
// Scratch layout of one piece of one CTA (128 rows x block_n fp32): 16-byte vectors in the order
// [32-column chunk][vector of the chunk (8)][row (128)], so that the epilogue's stores (thread =
// row) and the slice sums (consecutive threads = consecutive rows) are both coalesced.
__device__ __forceinline__ long long split_vec_offset(int col4, int row) {   // col4 = column / 4
  return (static_cast<long long>(col4) * kBlockM + row) * 16;
}

// silu(gate) * up on two fp32 values held as raw bits.
__device__ __forceinline__ uint32_t silu_mul(uint32_t gate_bits, uint32_t up_bits) {
  const float g = __uint_as_float(gate_bits);
  return __float_as_uint(__fdividef(g, 1.0f + __expf(-g)) * __uint_as_float(up_bits));
}

struct TileInfo {
  int rowblock, q, row0, rows, n0;
};
__device__ __forceinline__ TileInfo tile_info(const Sched& s, int t) {
  TileInfo ti;
  tile_to_coord(s, t, &ti.rowblock, &ti.q);
  ti.row0 = rowblock_row0(s, ti.rowblock);
  ti.rows = rowblock_rows(s, ti.rowblock);
  ti.n0 = ti.q * s.block_n;
  return ti;
}

// Where row `grow` of this rank's GEMM output lives.
template <int OP>
__device__ __forceinline__ __nv_bfloat16* output_row(const OpParams& p, int grow) {
  const Sched& s = p.sched;
  if (OP == OP_RS && s.world > 1 && !diag(p, 2)) {
    // ReduceScatter: the row belongs to owner o and goes straight into o's buffer, into the
    // slab reserved for this (producing) rank.  Remote when o != rank: posted NVLink writes.
    int o = grow / s.part_rows;
    if (o > s.world - 1) o = s.world - 1;
    const int i = grow - o * s.part_rows;
    return static_cast<__nv_bfloat16*>(p.peer_data[o]) +
           static_cast<long long>(s.rank * s.part_rows + i) * p.ldc;
  }
  return static_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(grow) * p.ldc;
}

// ------------------------------------------------------------------------------------------
// GEMM roles of a compute CTA (warps 0, 1, 2, 4-7)
// ------------------------------------------------------------------------------------------
// CG = 1: every CTA computes its own 128 x block_n tiles.
// CG = 2: CTAs run as pairs (a cluster of two).  The pair works on two tiles of the same column
// block at a time, one per CTA; each CTA loads its own A tile and HALF of the B tile, the leader
// (cluster rank 0) issues one 256 x block_n MMA per K step that reads both halves, and each CTA
// drains its own 128 accumulator rows.  This halves the shared-memory traffic for B.
// The two tiles need not be adjacent rows: consecutive tiles in visiting order share the column
// block (the row-block index runs fastest inside a raster group of even height).
template <int OP, int CG>
__device__ __forceinline__ void compute_roles(const CUtensorMap* tma_a, const CUtensorMap* tma_b,
                                              const OpParams& p, uint32_t smem_base,
                                              uint32_t bar_base, uint32_t epi_stage,
                                              uint32_t tmem_base, WaitCtx& wc, uint32_t epoch,
                                              volatile uint32_t* s_progress) {
  const Sched& s = p.sched;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_comp = gridDim.x - p.n_comm;
  const int crank = CG == 2 ? static_cast<int>(ptx::cluster_ctarank()) : 0;
  // First tile of this CTA; the stride is n_comp for both modes (pairs step by n_comp / 2).
  const int cta = CG == 2 ? (((static_cast<int>(blockIdx.x) - p.n_comm) & ~1) + crank)
                          : static_cast<int>(blockIdx.x) - p.n_comm;
  const int total = diag(p, 32) ? 0 : s.P * s.Q;   // diagnostics: exchange only
  const int bn = s.block_n;
  const int b_rows = bn / CG;                         // B rows (columns of C) this CTA loads
  const int stage_sz = kBlockM * kBlockK * 2 + b_rows * kBlockK * 2;
  auto bar = [&](int slot) { return bar_base + 8u * slot; };
  // Barriers the pair shares live in the leader CTA.
  auto lead = [&](int slot) { return CG == 2 ? ptx::map_to_cta(bar(slot), 0) : bar(slot); };
  constexpr bool kSignals = (OP == OP_RS || OP == OP_AR);
  SplitPlan split;
  split.full_rounds = 0; split.rem_units = 0; split.parts = 0;
  if (OP == OP_GEMM || OP == OP_AG) split = make_split<CG>(p, total, n_comp);
  // Diagnostics build: p.trace set = coarse counters (kernel and MMA-loop cycles); flag 256 adds
  // a cycle-counter read around every wait, which itself slows the MMA issue loop.
  const bool trc = kDiag && p.trace != nullptr;
  const bool tr = trc && diag(p, 256);

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    // Everything the per-k-block loop needs is copied into registers first: the parameter block
    // is read through a reference, and every barrier / TMA instruction below is a compiler
    // memory barrier, so a field left in the block would be re-read once per use.
    wc.where = (blockIdx.x << 8) | 0u;
    const int stages = p.stages;
    const bool b_mn = p.b_mn_major != 0;
    const bool no_loads = diag(p, 64), idle = diag(p, 1024);
    const uint32_t full0 = CG == 2 ? lead(BAR_FULL) : bar(BAR_FULL);   // + 8 * stage
    const uint32_t full0_local = bar(BAR_FULL), empty0 = bar(BAR_EMPTY);
    const uint32_t tx_bytes = static_cast<uint32_t>(CG * stage_sz);
    const int b_panels = b_rows / 64;
    // AllGather in K-range form: vectors per range (log2) and ranges per row
    const int ag_lg = OP == OP_AG ? p.ag_cv_log2 : 0;
    const int ag_ranges = ag_lg != 0 ? ((p.K / 8) + (1 << ag_lg) - 1) >> ag_lg : 0;
    const int ag_kb_shift = ag_lg > 3 ? ag_lg - 3 : 0;   // k-blocks per range, log2 (a range is >= 8 vectors)
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    long long tr_empty = 0, tr_gather = 0;
    WorkItem w;
    for (int it = 0; ok && work_item<CG>(p, split, total, n_comp, cta, it, w); ++it) {
      const int t = w.t;
      const TileInfo ti = tile_info(s, t);
      if (OP == OP_AG && lane == 0) *s_progress = static_cast<uint32_t>(t);
      uint32_t landed = 0xffffffffu;   // K-ranges of this tile's rows known to have landed here
      const uint32_t* range_flags = nullptr;
      if (OP == OP_AG && s.world > 1 && rowblock_shard(s, ti.rowblock) != s.rank) {
        static_assert(kGatherSub == 32, "one group / range flag per producer lane");
        const uint32_t* f = p.sync + SW_FLAGS + gather_flag_index(ti.rowblock, lane);
        const long long c0 = diag_clock(tr);
        if (ag_lg == 0) {
          // Rows of a remote shard: wait until the sender has landed all 4-row groups here.
          const bool mine = bounded_wait<true>(wc, [&] { return ptx::ld_acquire_sys(f) == epoch; },
                                               ST_TIMEOUT_GATHER, ti.rowblock, lane);
          ok = __all_sync(0xffffffffu, mine);
        } else {
          // K-range form: note which ranges are here already; the K loop waits for the others
          // one by one as it reaches them.
          range_flags = f - lane;
          landed = __ballot_sync(0xffffffffu, lane >= ag_ranges || ptx::ld_acquire_sys(f) == epoch);
        }
        tr_gather += diag_clock(tr) - c0;
        ptx::fence_proxy_async();  // rows stored by a peer GPU are about to be read by TMA
        if (!ok) break;
      }
      if (lane == 0 && !idle) {
        const int row0 = ti.row0;
        const int nb0 = ti.n0 + crank * b_rows;   // first B row (C column) this CTA loads
        int kx = w.kb0 * kBlockK;                  // element offset of the k-block
        for (int kb = w.kb0; kb < w.kb1; ++kb, kx += kBlockK) {
          if (OP == OP_AG && landed != 0xffffffffu) {
            const int c = kb >> ag_kb_shift;
            if (((landed >> c) & 1u) == 0u) {
              const uint32_t* f = range_flags + c;
              const long long g0 = diag_clock(tr);
              if (!bounded_wait<true>(wc, [&] { return ptx::ld_acquire_sys(f) == epoch; },
                                      ST_TIMEOUT_GATHER, ti.rowblock, c)) { ok = false; break; }
              tr_gather += diag_clock(tr) - g0;
              ptx::fence_proxy_async();
              landed |= 1u << c;
            }
          }
          const long long c0 = diag_clock(tr);
          if (!wait_mbar(wc, empty0 + 8u * stage, phase ^ 1u, 0x100u + stage)) { ok = false; break; }
          tr_empty += diag_clock(tr) - c0;
          const uint32_t a_dst = smem_base + stage * stage_sz;
          const uint32_t b_dst = a_dst + kBlockM * kBlockK * 2;
          const uint32_t full = full0 + 8u * stage;
          if (kDiag && no_loads) {
            // diagnostics: no operand loads, the MMAs run on whatever the stage holds
            if (crank == 0) ptx::mbar_arrive(full0_local + 8u * stage);
          } else if (CG == 1) {
            ptx::mbar_expect_tx(full, tx_bytes);
            ptx::tma_load_2d(a_dst, tma_a, full, kx, row0);
            if (!b_mn) {
              ptx::tma_load_2d(b_dst, tma_b, full, kx, nb0);
            } else {
              for (int c = 0; c < b_panels; ++c)
                ptx::tma_load_2d(b_dst + c * 8192, tma_b, full, nb0 + c * 64, kx);
            }
          } else {
            // Both CTAs' bytes are counted on the leader's barrier; only the leader arrives.
            if (crank == 0) ptx::mbar_expect_tx(full0_local + 8u * stage, tx_bytes);
            ptx::tma_load_2d_pair(a_dst, tma_a, full, kx, row0);
            if (!b_mn) {
              ptx::tma_load_2d_pair(b_dst, tma_b, full, kx, nb0);
            } else {
              for (int c = 0; c < b_panels; ++c)
                ptx::tma_load_2d_pair(b_dst + c * 8192, tma_b, full, nb0 + c * 64, kx);
            }
          }
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
      }
      ok = __all_sync(0xffffffffu, ok);
    }
    if (OP == OP_AG && lane == 0) *s_progress = 0x7fffffffu;   // nothing left to pace against
    if (tr && lane == 0) {
      p.trace[blockIdx.x * 16 + 2] = tr_empty;
      p.trace[blockIdx.x * 16 + 3] = tr_gather;
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (one warp, one elected lane issues) ----------------
    // This loop feeds the tensor pipe and is bound by the latency of its own instruction stream:
    // a k-block is four MMAs (512 tensor cycles at N = 256), and measured on B200 every cycle the
    // issuing lane spends between two MMAs is a cycle the pipe idles (a loop that re-read
    // parameters and built descriptors per MMA ran 765 cycles per k-block, this one 512-545).
    // So: all loop state lives in registers (see the producer); the whole warp runs the loop
    // with uniform control flow (wait results are combined with a vote), which lets the compiler
    // keep that state in uniform registers; and each k-block's MMAs and commits are ONE statement
    // that elects its issuing lane and advances the descriptors by adding to their low word.
    wc.where = (blockIdx.x << 8) | 1u;
    if (crank == 0) {
      const int stages = p.stages;
      const bool b_mn = p.b_mn_major != 0;
      const uint32_t idesc = ptx::make_idesc_bf16(bn, b_mn ? 1u : 0u, 128u * CG);
      const uint32_t desc_hi = static_cast<uint32_t>(ptx::make_smem_desc_sw128(0, 0, 1024) >> 32);
      const uint32_t a_lo0 = static_cast<uint32_t>(ptx::make_smem_desc_sw128(smem_base, 16, 1024));
      const uint32_t b_lo0 = static_cast<uint32_t>(
          ptx::make_smem_desc_sw128(smem_base + kBlockM * kBlockK * 2, b_mn ? 8192 : 16, 1024));
      const uint32_t b_kstep = b_mn ? (2048u >> 4) : (32u >> 4);
      const uint32_t stage_step = static_cast<uint32_t>(stage_sz) >> 4;
      const uint32_t full0 = bar(BAR_FULL);
      const uint32_t empty_a = CG == 2 ? ptx::map_to_cta(bar(BAR_EMPTY), 0) : bar(BAR_EMPTY);
      const uint32_t empty_b = CG == 2 ? ptx::map_to_cta(bar(BAR_EMPTY), 1) : 0u;
      const uint32_t tfull_a = CG == 2 ? ptx::map_to_cta(bar(BAR_TFULL), 0) : bar(BAR_TFULL);
      const uint32_t tfull_b = CG == 2 ? ptx::map_to_cta(bar(BAR_TFULL), 1) : 0u;
      // the TMEM base was read from shared memory; a warp reduction makes it a uniform value
      const uint32_t d_base = __reduce_or_sync(0xffffffffu, tmem_base);
      const bool no_mma = diag(p, 128), no_full_wait = diag(p, 512 | 1024), no_release = diag(p, 1024);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      uint32_t a_lo = a_lo0, b_lo = b_lo0;
      bool ok = true;
      long long tr_tiles = 0;
      const long long tr_begin = diag_clock(trc);
      WorkItem w;
      for (int it = 0; work_item<CG>(p, split, total, n_comp, cta, it, w); ++it) {
        if (!__all_sync(0xffffffffu,
                        wait_mbar(wc, bar(BAR_TEMPTY + acc), acc_phase ^ 1u, 0x200u + acc)))
          break;
        ++tr_tiles;
        ptx::tc_fence_after();
        const uint32_t d_tmem = d_base + acc * 256;
        uint32_t accumulate = 0u;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!(kDiag && no_full_wait) &&
              !__all_sync(0xffffffffu, wait_mbar(wc, full0 + 8u * stage, phase, 0x300u + stage))) {
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          if (kDiag && no_mma)
            ptx::umma_commit_elect<CG>(empty_a + 8u * stage, empty_b + 8u * stage);
          else
            ptx::umma_kblock<CG>(d_tmem, a_lo, b_lo, b_kstep, desc_hi, idesc, accumulate,
                                 empty_a + 8u * stage, empty_b + 8u * stage,
                                 !(kDiag && no_release));
          accumulate = 1u;
          a_lo += stage_step;
          b_lo += stage_step;
          if (++stage == stages) { stage = 0; phase ^= 1u; a_lo = a_lo0; b_lo = b_lo0; }
        }
        if (!ok) break;
        // accumulator complete (each CTA of a pair holds its own 128 rows)
        ptx::umma_commit_elect<CG>(tfull_a + 8u * acc, tfull_b + 8u * acc);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (trc && lane == 0) {
        unsigned long long* o = p.trace + blockIdx.x * 16;
        o[6] = clock64() - tr_begin; o[9] = tr_tiles;
      }
    }
  } else if (warp == 2) {
    // ---------------- tile publisher (RS / AR) ----------------
    wc.where = (blockIdx.x << 8) | 2u;
    if (kSignals && s.world > 1 && lane == 0) {
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = cta; t < total; t += n_comp) {
        const TileInfo ti = tile_info(s, t);
        if (!wait_mbar(wc, bar(BAR_STORED + acc), acc_phase, 0x400u + acc)) break;
        // The tile's rows have been stored (possibly to other GPUs); make them visible
        // system-wide, then tell every owner whose rows intersect the tile.  (Not needed when
        // the rows went into slabs that carry the epoch next to every data word.)
        if (!(OP == OP_AR && s.ar_push == 2)) {
          ptx::fence_acq_rel_sys();
          int lo, hi;
          rowblock_owners(s, ti.rowblock, &lo, &hi);
          const long long idx = SW_FLAGS + tile_flag_index(s, s.rank, ti.rowblock, ti.q);
          for (int o = lo; o <= hi; ++o) ptx::st_relaxed_sys(p.peer_sync[o] + idx, epoch);
        }
        stamp_max(p, 1);
        if (CG == 1) ptx::mbar_arrive(bar(BAR_TEMPTY + acc));
        else ptx::mbar_arrive_cluster(lead(BAR_TEMPTY + acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp >= 4) {
    // ---------------- epilogue ----------------
    // TMEM lane = output row, so a thread holds one row of 64 consecutive columns (128 B).
    // The warp transposes through a private 4 KB shared-memory buffer (16-byte pieces, XOR
    // swizzled) so that every store instruction writes four complete 128-byte row segments.
    wc.where = (blockIdx.x << 8) | 4u;
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    const uint32_t stage_buf = epi_stage + quarter * 4096;
    int acc = 0;
    uint32_t acc_phase = 0;
    const int sub_row = lane >> 3, piece = lane & 7;
    uint32_t entered_mask = 1u << s.rank;  // owners known to have entered this launch
    long long tr_tfull = 0, tr_busy = 0;
    // loop state in registers (see the producer)
    const int N = s.N, world = s.world, rank = s.rank, part_rows = s.part_rows;
    const long long ldc = p.ldc;
    __nv_bfloat16* const c_local = static_cast<__nv_bfloat16*>(p.C);
    __nv_bfloat16* const c_copy =
        (OP == OP_AR && world == 1) ? static_cast<__nv_bfloat16*>(p.peer_out[0]) : nullptr;
    // ReduceScatter through NVSwitch (opt-in): partial tiles stay in this rank's own buffer and
    // the owner sums all replicas with one switch-side reduction per vector.
    const bool rs_in_switch = OP == OP_RS && p.use_nvls && p.mc_data != nullptr;
    const bool to_owner = OP == OP_RS && world > 1 && !rs_in_switch && !diag(p, 2);
    const int slab_mode = OP == OP_AR ? s.ar_push : 0;    // second copy into the owner's slab
    const bool to_slab = slab_mode != 0;
    // bytes per slab row: plain bf16, or (mode 2) every 32-bit word followed by the epoch
    const long long slab_pitch = static_cast<long long>(N) * (slab_mode == 2 ? 4 : 2);
    // SwiGLU epilogue (plain GEMM and AllGather+GEMM): half as many output columns
    const bool glu = (OP == OP_GEMM || OP == OP_AG) && p.epilogue == EPI_SWIGLU;
    const int out_bn = glu ? bn / 2 : bn, n_out = glu ? N / 2 : N;
    const uint32_t tfull0 = bar(BAR_TFULL), stored0 = bar(BAR_STORED);
    const uint32_t tempty0 = CG == 2 ? lead(BAR_TEMPTY) : bar(BAR_TEMPTY);
    WorkItem w;
    for (int wi = 0; work_item<CG>(p, split, total, n_comp, cta, wi, w); ++wi) {
      const int t = w.t;
      const TileInfo ti = tile_info(s, t);
      if ((OP == OP_GEMM || OP == OP_AG) && w.piece >= 0) {
        // ---- a piece of a tail tile: fp32 partial -> scratch; then sum a slice of the tile ----
        if (!wait_mbar(wc, tfull0 + 8u * acc, acc_phase, 0x500u + acc)) break;
        ptx::tc_fence_after();
        const uint32_t t_base = tmem_base + acc * 256 + (static_cast<uint32_t>(quarter * 32) << 16);
        const long long slot_bytes = static_cast<long long>(kBlockM) * bn * 4;
        char* const scratch = reinterpret_cast<char*>(p.split_scratch);
        char* const mine = scratch + (static_cast<long long>(w.piece) * CG + crank) * slot_bytes;
        const int my_tile_row = quarter * 32 + lane;
        for (int c = 0; c < bn; c += 32) {
          uint32_t r0[32];
          ptx::tmem_ld_32x32(t_base + c, r0);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 8; ++v)
            ptx::st_global_v4(mine + split_vec_offset(c / 4 + v, my_tile_row),
                              make_uint4(r0[4 * v], r0[4 * v + 1], r0[4 * v + 2], r0[4 * v + 3]));
        }
        ptx::tc_fence_before();
        __threadfence();                                   // the partial is visible device-wide
        __syncwarp();
        const int tail_tile = w.piece / split.parts, part = w.piece % split.parts;
        uint32_t* const counter = p.split_counters + tail_tile * CG + crank;
        // The CTA's arrival is announced once all four epilogue warps have stored their rows.
        // They meet through a shared counter and a bounded wait, never through a hardware
        // barrier: a warp that gave up on an earlier wait must not leave the others stuck.
        if (lane == 0) atomicAdd(const_cast<uint32_t*>(s_progress) + 2, 1u);
        if (warp == 4 && lane == 0) {
          volatile uint32_t* stored = s_progress + 2;
          if (bounded_wait<true>(wc, [&] { return *stored >= 4u; }, ST_TIMEOUT_PIPE, 0x701u,
                                 static_cast<uint32_t>(w.piece)))
            atomicAdd(counter, 1u);
        }
        // every piece of this tile half has arrived?
        {
          const uint32_t want = static_cast<uint32_t>(split.parts);
          const bool ok = bounded_wait<true>(wc, [&] { return ptx::ld_acquire_gpu(counter) >= want; },
                                             ST_TIMEOUT_PIPE, 0x700u, static_cast<uint32_t>(w.piece));
          if (!__all_sync(0xffffffffu, ok)) break;
        }
        // Sum rows [part * R, part * R + R) of this CTA's 128 over all pieces, in piece order.
        const int R = (kBlockM + split.parts - 1) / split.parts;
        const int r_lo = part * R;
        int r_hi = r_lo + R;
        if (r_hi > ti.rows) r_hi = ti.rows;
        const int nr = r_hi - r_lo;
        if (nr > 0) {
          const int n_cv = out_bn / 4;                     // output vectors (4 columns) per row
          const char* const first = scratch + (static_cast<long long>(tail_tile) * split.parts * CG + crank) * slot_bytes;
          const long long piece_stride = slot_bytes * CG;
          const int tid = (warp - 4) * 32 + lane;
          const int n0_out = glu ? ti.n0 / 2 : ti.n0;
          for (int id = tid; id < n_cv * nr; id += 128) {
            const int row = r_lo + id % nr, cv = id / nr;
            const int col = n0_out + cv * 4;
            if (col >= n_out) continue;
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, u0 = 0.f, u1 = 0.f, u2 = 0.f, u3 = 0.f;
            const char* q = first + split_vec_offset(cv, row);
            for (int pc = 0; pc < split.parts; ++pc, q += piece_stride) {
              const float4 x = __ldcg(reinterpret_cast<const float4*>(q));
              a0 += x.x; a1 += x.y; a2 += x.z; a3 += x.w;
              if (glu) {
                const float4 y = __ldcg(reinterpret_cast<const float4*>(q + split_vec_offset(n_cv, 0)));
                u0 += y.x; u1 += y.y; u2 += y.z; u3 += y.w;
              }
            }
            if (glu) {
              a0 = __uint_as_float(silu_mul(__float_as_uint(a0), __float_as_uint(u0)));
              a1 = __uint_as_float(silu_mul(__float_as_uint(a1), __float_as_uint(u1)));
              a2 = __uint_as_float(silu_mul(__float_as_uint(a2), __float_as_uint(u2)));
              a3 = __uint_as_float(silu_mul(__float_as_uint(a3), __float_as_uint(u3)));
            }
            uint2 o;
            o.x = ptx::pack_bf16x2(a0, a1);
            o.y = ptx::pack_bf16x2(a2, a3);
            *reinterpret_cast<uint2*>(c_local + static_cast<long long>(ti.row0 + row) * ldc + col) = o;
          }
        }
        __syncwarp();
        if (lane == 0) {
          if (CG == 1) ptx::mbar_arrive(tempty0 + 8u * acc);
          else ptx::mbar_arrive_cluster(tempty0 + 8u * acc);
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
        continue;
      }
      if (OP == OP_RS && world > 1) {
        // Rows of this tile go into their owners' buffers: an owner's buffer may be written
        // only once that owner has entered this launch (its previous reduce has ended).
        int lo, hi;
        rowblock_owners(s, ti.rowblock, &lo, &hi);
        bool ok = true;
        for (int o = lo; o <= hi && ok; ++o) {
          if (entered_mask & (1u << o)) continue;
          const uint32_t* f = p.sync + SW_ENTRY + o;
          ok = bounded_wait<true>(wc, [&] { return reached(ptx::ld_acquire_sys(f), epoch); },
                                  ST_TIMEOUT_ENTRY, o, epoch);
          entered_mask |= 1u << o;
        }
        if (!__all_sync(0xffffffffu, ok)) break;
      }
      // Destination of the eight rows this lane stores per 64-column chunk (row it*4 + sub_row
      // of the warp's 32): the local C, or for ReduceScatter the owner's buffer, in the slab
      // reserved for this (producing) rank -- remote when owner != rank: posted NVLink writes.
      __nv_bfloat16* row_ptr[8];
      char* slab_ptr[OP == OP_AR ? 8 : 1];
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int r_in_tile = quarter * 32 + it * 4 + sub_row;
        const int grow = ti.row0 + r_in_tile;
        if (OP == OP_AR) {
          slab_ptr[it] = nullptr;
          if (to_slab && r_in_tile < ti.rows) {
            int o = grow / part_rows;
            if (o > world - 1) o = world - 1;
            slab_ptr[it] = reinterpret_cast<char*>(p.peer_sync[o]) + kArSlabByteOffset +
                           static_cast<long long>(rank * part_rows + (grow - o * part_rows)) * slab_pitch;
          }
        }
        if (r_in_tile >= ti.rows) {
          row_ptr[it] = nullptr;
        } else if (to_owner) {
          int o = grow / part_rows;
          if (o > world - 1) o = world - 1;
          row_ptr[it] = static_cast<__nv_bfloat16*>(p.peer_data[o]) +
                        static_cast<long long>(rank * part_rows + (grow - o * part_rows)) * ldc;
        } else {
          row_ptr[it] = c_local + static_cast<long long>(grow) * ldc;
        }
      }
      const int n0_out = glu ? ti.n0 / 2 : ti.n0;
      const long long c0 = diag_clock(tr);
      if (!wait_mbar(wc, tfull0 + 8u * acc, acc_phase, 0x500u + acc)) break;
      const long long c1 = diag_clock(tr);
      tr_tfull += c1 - c0;
      ptx::tc_fence_after();
      const uint32_t t_base = tmem_base + acc * 256 + (static_cast<uint32_t>(quarter * 32) << 16);
      const uint32_t my_row = stage_buf + lane * 128;
      for (int c = 0; c < out_bn; c += 64) {
        const bool two = c + 32 < out_bn;
        uint32_t r0[32], r1[32];
        ptx::tmem_ld_32x32(t_base + c, r0);
        if (two) ptx::tmem_ld_32x32(t_base + c + 32, r1);
        if (glu) {
          // Gated activation: the tile's first half of columns is the gate, the second half the
          // up projection of the same output columns; out = silu(gate) * up, in fp32.
          uint32_t u[32];
          ptx::tmem_ld_32x32(t_base + out_bn + c, u);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) r0[j] = silu_mul(r0[j], u[j]);
          ptx::tmem_ld_32x32(t_base + out_bn + c + 32, u);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) r1[j] = silu_mul(r1[j], u[j]);
        }
        ptx::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 v;
          v.x = ptx::pack_bf16x2(__uint_as_float(r0[j * 8 + 0]), __uint_as_float(r0[j * 8 + 1]));
          v.y = ptx::pack_bf16x2(__uint_as_float(r0[j * 8 + 2]), __uint_as_float(r0[j * 8 + 3]));
          v.z = ptx::pack_bf16x2(__uint_as_float(r0[j * 8 + 4]), __uint_as_float(r0[j * 8 + 5]));
          v.w = ptx::pack_bf16x2(__uint_as_float(r0[j * 8 + 6]), __uint_as_float(r0[j * 8 + 7]));
          ptx::st_shared_v4(my_row + ((j ^ (lane & 7)) << 4), v);
        }
        if (two) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 v;
            v.x = ptx::pack_bf16x2(__uint_as_float(r1[j * 8 + 0]), __uint_as_float(r1[j * 8 + 1]));
            v.y = ptx::pack_bf16x2(__uint_as_float(r1[j * 8 + 2]), __uint_as_float(r1[j * 8 + 3]));
            v.z = ptx::pack_bf16x2(__uint_as_float(r1[j * 8 + 4]), __uint_as_float(r1[j * 8 + 5]));
            v.w = ptx::pack_bf16x2(__uint_as_float(r1[j * 8 + 6]), __uint_as_float(r1[j * 8 + 7]));
            ptx::st_shared_v4(my_row + (((j + 4) ^ (lane & 7)) << 4), v);
          }
        }
        __syncwarp();
        const int col = n0_out + c + piece * 8;
        const bool col_ok = (piece < (two ? 8 : 4)) && (col + 8 <= n_out);
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int r = it * 4 + sub_row;            // row inside this warp's 32 rows
          if (col_ok && row_ptr[it] != nullptr) {
            const uint4 v = ptx::ld_shared_v4(stage_buf + r * 128 + ((piece ^ (r & 7)) << 4));
            ptx::st_global_v4(row_ptr[it] + col, v);
            if (OP == OP_AR && c_copy != nullptr)   // one GPU: the partial product is the result
              ptx::st_global_v4(c_copy + (row_ptr[it] - c_local) + col, v);
            if (OP == OP_AR && slab_ptr[it] != nullptr) {
              if (slab_mode == 2) {
                // data word, epoch, data word, epoch: the reader needs no separate flag
                ptx::st_global_v4(slab_ptr[it] + col * 4, make_uint4(v.x, epoch, v.y, epoch));
                ptx::st_global_v4(slab_ptr[it] + col * 4 + 16, make_uint4(v.z, epoch, v.w, epoch));
              } else {
                ptx::st_global_v4(slab_ptr[it] + col * 2, v);
              }
            }
          }
        }
        __syncwarp();
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (CG == 1) ptx::mbar_arrive(tempty0 + 8u * acc);
        else ptx::mbar_arrive_cluster(tempty0 + 8u * acc);
        if (kSignals && world > 1) ptx::mbar_arrive(stored0 + 8u * acc);
      }
      tr_busy += diag_clock(tr) - c1;
      if (kDiag && t == cta && blockIdx.x == 0 && warp == 4 && lane == 0) stamp(p, 7);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    // Latency-bound AllReduce: the exchange warp holds back until this CTA's tiles are stored
    // (its polling would compete with the operand stream for L2 bandwidth, and all ranks run the
    // same GEMM, so the peers' rows cannot be there much earlier anyway).
    if (OP == OP_AR && warp == 4 && lane == 0) *s_progress = 1u;
    if (tr && warp == 4 && lane == 0) {
      p.trace[blockIdx.x * 16 + 7] = tr_tfull;
      p.trace[blockIdx.x * 16 + 8] = tr_busy;
    }
  }
}

// ------------------------------------------------------------------------------------------
// Exchange workers (one warp each)
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void accumulate_bf16x8(float (&acc)[8], const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i + 0] += __uint_as_float(w[i] << 16);
    acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
  }
}

// The span loops below run on ONE warp next to the GEMM, so their own instruction count decides
// how fast bytes move: all index arithmetic is 32-bit, addresses advance by constants, and a step
// whose vectors are all in range takes a branch-free path.
//
// Ring geometry shared by the push loops: a ring of R slots per lane (slot = 32 lanes x 16 bytes,
// 512 bytes) is used as NS steps of VP slots.  Vector e of a lane (the lane's e-th 16 bytes, i.e.
// vector e * 32 + lane of the span) lives in slot e % R = (step % NS) * VP + j.  One cp.async
// commit group per step keeps the number of groups in flight small (<= 12) however deep the ring.
template <int R>
struct PushRing {
  static constexpr int VP = R >= 64 ? 8 : 4;   // vectors per lane per step
  static constexpr int NS = R / VP;            // steps in the ring
  static constexpr int kStepBytes = VP * 512;
  static_assert(NS >= 3 && NS <= 12 && NS * VP == R, "ring geometry");
};

// Loads of a push loop: `issue()` starts the next step's cp.async copies (or an empty group past
// the end) and advances; the caller consumes step st after cp_async_wait<NS - 1 (or - 2)>.
template <int R>
struct PushLoader {
  using G = PushRing<R>;
  const char* src;     // lane's next source address
  uint32_t ring_lane;  // ring base + lane * 16
  int n_mine, n_steps, step, slot;
  bool skip;
  __device__ __forceinline__ PushLoader(const char* s, uint32_t ring, int n_vec, int lane, bool skip_)
      : src(s + lane * 16), ring_lane(ring + lane * 16u),
        n_mine(n_vec > lane ? (n_vec - 1 - lane) / 32 + 1 : 0), step(0), slot(0), skip(skip_) {
    n_steps = (n_mine + G::VP - 1) / G::VP;
  }
  __device__ __forceinline__ uint32_t slot_addr(int ring_step) const {
    return ring_lane + static_cast<uint32_t>(ring_step) * G::kStepBytes;
  }
  __device__ __forceinline__ void issue() {
    if (step < n_steps && !skip) {
      const uint32_t sb = slot_addr(slot);
      const int left = n_mine - step * G::VP;
      if (left >= G::VP) {
#pragma unroll
        for (int j = 0; j < G::VP; ++j) ptx::cp_async_16(sb + j * 512, src + j * 512);
      } else {
#pragma unroll
        for (int j = 0; j < G::VP; ++j)
          if (j < left) ptx::cp_async_16(sb + j * 512, src + j * 512);
      }
    }
    ptx::cp_async_commit();
    src += G::kStepBytes;
    ++step;
    if (++slot == G::NS) slot = 0;
  }
};

// AllGather item: copy `n_vec` 16-byte vectors from the own shard to the same offset of up to
// kMaxWorld - 1 destinations (peers' buffers; or one destination: a peer or the multicast alias)
// through the lane-private ring.  Every vector is loaded once.
template <int R, int ND>
__device__ __forceinline__ void push_span(const char* src, char* const (&dst_in)[ND], int n_dst,
                                          int n_vec, bool nvls, uint32_t ring, int lane, int dbg) {
  using G = PushRing<R>;
  PushLoader<R> ld(src, ring, n_vec, lane, (dbg & 8) != 0);
  char* dst[ND];
#pragma unroll
  for (int d = 0; d < ND; ++d) dst[d] = d < n_dst ? dst_in[d] + lane * 16 : nullptr;
#pragma unroll 1
  for (int i = 0; i < G::NS - 1; ++i) ld.issue();
  int slot = 0;
#pragma unroll 1
  for (int st = 0; st < ld.n_steps; ++st) {
    ld.issue();
    ptx::cp_async_wait<G::NS - 1>();
    const uint32_t sb = ld.slot_addr(slot);
    const int left = ld.n_mine - st * G::VP;
    uint4 v[G::VP];
#pragma unroll
    for (int j = 0; j < G::VP; ++j) v[j] = ptx::ld_shared_v4(sb + j * 512);
    if (!(dbg & 16)) {
#pragma unroll
      for (int d = 0; d < ND; ++d) {
        if (d >= n_dst) break;
        if (left >= G::VP) {
#pragma unroll
          for (int j = 0; j < G::VP; ++j) {
            if (nvls) ptx::multimem_st_v4(dst[d] + j * 512, v[j]);
            else ptx::st_global_v4(dst[d] + j * 512, v[j]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < G::VP; ++j) {
            if (j >= left) break;
            if (nvls) ptx::multimem_st_v4(dst[d] + j * 512, v[j]);
            else ptx::st_global_v4(dst[d] + j * 512, v[j]);
          }
        }
        dst[d] += G::kStepBytes;
      }
    }
    if (++slot == G::NS) slot = 0;
  }
  ptx::cp_async_wait<0>();
}

// AllGather item in K-range form: `rows` rows of one row-block, each row's `valid_cv` (<= 2^lg_cv)
// 16-byte vectors starting at the same column, from the own shard to the same offsets of one
// destination.  Vector v of the item is (row v >> lg_cv, column v & (2^lg_cv - 1)); a warp step
// therefore covers whole 128..512-byte row segments.  Same ring discipline as push_span.
template <int R>
__device__ __forceinline__ void push_chunk(const char* src, char* dst, int rows, long long row_bytes,
                                           int lg_cv, int valid_cv, uint32_t ring, int lane) {
  using G = PushRing<R>;
  const int col_mask = (1 << lg_cv) - 1;
  const int n_vec = rows << lg_cv;
  const int n_mine = n_vec > lane ? (n_vec - 1 - lane) / 32 + 1 : 0;
  const int n_steps = (n_mine + G::VP - 1) / G::VP;
  const uint32_t ring_lane = ring + lane * 16u;
  // byte offset of this lane's e-th vector, or -1 where the row has no such column
  auto offset_of = [=](int e) -> long long {
    const int v = e * 32 + lane;
    const int col = v & col_mask;
    if (e >= n_mine || col >= valid_cv) return -1;
    return static_cast<long long>(v >> lg_cv) * row_bytes + col * 16;
  };
  int ld_step = 0, ld_slot = 0;
  auto issue = [&]() {
    if (ld_step < n_steps) {
      const uint32_t sb = ring_lane + static_cast<uint32_t>(ld_slot) * G::kStepBytes;
#pragma unroll
      for (int j = 0; j < G::VP; ++j) {
        const long long off = offset_of(ld_step * G::VP + j);
        if (off >= 0) ptx::cp_async_16(sb + j * 512, src + off);
      }
    }
    ptx::cp_async_commit();
    ++ld_step;
    if (++ld_slot == G::NS) ld_slot = 0;
  };
#pragma unroll 1
  for (int i = 0; i < G::NS - 1; ++i) issue();
  int slot = 0;
#pragma unroll 1
  for (int st = 0; st < n_steps; ++st) {
    issue();
    ptx::cp_async_wait<G::NS - 1>();
    const uint32_t sb = ring_lane + static_cast<uint32_t>(slot) * G::kStepBytes;
    uint4 v[G::VP];
    long long off[G::VP];
#pragma unroll
    for (int j = 0; j < G::VP; ++j) {
      off[j] = offset_of(st * G::VP + j);
      v[j] = ptx::ld_shared_v4(sb + j * 512);
    }
#pragma unroll
    for (int j = 0; j < G::VP; ++j)
      if (off[j] >= 0) ptx::st_global_v4(dst + off[j], v[j]);
    if (++slot == G::NS) slot = 0;
  }
  ptx::cp_async_wait<0>();
}

// Same copy to one destination, but every step (VP x 32 vectors = one contiguous range in both
// the ring and the destination) leaves as ONE bulk store issued by lane 0: fewer, larger write
// requests on NVLink.
template <int R>
__device__ __forceinline__ void push_span_bulk(const char* src, char* dst, int n_vec,
                                               uint32_t ring, int lane) {
  using G = PushRing<R>;
  PushLoader<R> ld(src, ring, n_vec, lane, false);
  const int n_steps = (n_vec + G::VP * 32 - 1) / (G::VP * 32);          // same for every lane
  // The slots of step st are refilled by step st + NS - 2, issued after the bulk store of step
  // st - 1 ... so one ring step is always either being stored or free: NS - 2 steps in flight.
#pragma unroll 1
  for (int i = 0; i < G::NS - 2; ++i) ld.issue();
  int slot = 0;
#pragma unroll 1
  for (int st = 0; st < n_steps; ++st) {
    // the step about to be refilled was stored two iterations ago: its store must have read it
    if (lane == 0) ptx::bulk_wait_read<1>();
    __syncwarp();
    ld.issue();
    ptx::cp_async_wait<G::NS - 2>();
    ptx::fence_proxy_async();       // cp.async wrote the ring; the bulk store reads it
    __syncwarp();
    if (lane == 0) {
      int vecs = n_vec - st * (G::VP * 32);
      if (vecs > G::VP * 32) vecs = G::VP * 32;
      ptx::bulk_s2g(dst, ring + static_cast<uint32_t>(slot) * G::kStepBytes,
                    static_cast<uint32_t>(vecs * 16));
      ptx::bulk_commit();
    }
    dst += G::kStepBytes;
    if (++slot == G::NS) slot = 0;
  }
  ptx::cp_async_wait<0>();
  if (lane == 0) {
    ptx::bulk_wait_all<0>();   // every byte has been written before the flag goes out
    ptx::fence_proxy_async();
  }
  __syncwarp();
}

struct ReduceSpan {
  const char* src[kMaxWorld];  // W copies of the same byte range
  char* dst[kMaxWorld];        // RS: dst[0] only; AR: every rank's output
  char* mc_dst;                // AR through NVSwitch multicast (or nullptr)
  int n_vec;                   // 16-byte vectors in the range
};

// Reduce item: sum W copies of a range.  Each lane owns every 32nd vector; the ring holds NS
// steps of VP vectors x WT copies (slot of (step, j, copy) = ((step % NS) * VP + j) * WT + copy),
// one cp.async commit group per step, NS-1 steps in flight.  fp32 accumulation in fixed rank
// order 0..W-1.
template <int OP, int WT, int R>
__device__ __forceinline__ void reduce_span(const ReduceSpan& sp, int W, uint32_t ring, int lane) {
  constexpr int VP = (R / (WT * 8)) >= 1 ? R / (WT * 8) : 1;   // vectors per lane per step
  constexpr int NS = R / (WT * VP);                             // steps in the ring
  constexpr int kStepBytes = VP * WT * 512;
  static_assert(NS >= 2 && NS <= 12, "ring geometry");
  const int n_mine = sp.n_vec > lane ? (sp.n_vec - 1 - lane) / 32 + 1 : 0;
  const int n_steps = (n_mine + VP - 1) / VP;
  const uint32_t ring_lane = ring + lane * 16u;
  const char* src[WT];
#pragma unroll
  for (int c = 0; c < WT; ++c) src[c] = c < W ? sp.src[c] + lane * 16 : nullptr;
  int i_step = 0, i_slot = 0;
  auto issue = [&]() {
    if (i_step < n_steps) {
      const uint32_t sb = ring_lane + static_cast<uint32_t>(i_slot) * kStepBytes;
      const int left = n_mine - i_step * VP;
#pragma unroll
      for (int j = 0; j < VP; ++j) {
        if (j >= left) break;
#pragma unroll
        for (int c = 0; c < WT; ++c)
          if (c < W) ptx::cp_async_16(sb + (j * WT + c) * 512, src[c] + j * 512);
      }
    }
    ptx::cp_async_commit();
#pragma unroll
    for (int c = 0; c < WT; ++c) src[c] += VP * 512;
    ++i_step;
    if (++i_slot == NS) i_slot = 0;
  };
  long long off = lane * 16;   // byte offset of the lane's vector j = 0 of the current step
#pragma unroll 1
  for (int i = 0; i < NS - 1; ++i) issue();
  int slot = 0;
#pragma unroll 1
  for (int st = 0; st < n_steps; ++st) {
    issue();
    ptx::cp_async_wait<NS - 1>();
    const uint32_t sb = ring_lane + static_cast<uint32_t>(slot) * kStepBytes;
    const int left = n_mine - st * VP;
#pragma unroll
    for (int j = 0; j < VP; ++j) {
      if (j >= left) break;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < WT; ++c)
        if (c < W) accumulate_bf16x8(acc, ptx::ld_shared_v4(sb + (j * WT + c) * 512));
      uint4 r;
      r.x = ptx::pack_bf16x2(acc[0], acc[1]);
      r.y = ptx::pack_bf16x2(acc[2], acc[3]);
      r.z = ptx::pack_bf16x2(acc[4], acc[5]);
      r.w = ptx::pack_bf16x2(acc[6], acc[7]);
      const long long o = off + j * 512;
      if (OP == OP_RS) {
        ptx::st_global_v4(sp.dst[0] + o, r);
      } else if (sp.mc_dst != nullptr) {
        ptx::multimem_st_v4(sp.mc_dst + o, r);
      } else {
#pragma unroll
        for (int d = 0; d < WT; ++d)
          if (d < W && sp.dst[d] != nullptr) ptx::st_global_v4(sp.dst[d] + o, r);
      }
    }
    off += VP * 512;
    if (++slot == NS) slot = 0;
  }
  ptx::cp_async_wait<0>();
}

// AllReduce through NVSwitch: one multimem load returns the fp32-accumulated sum of all replicas.
// kLocalDst: the sums go to this rank's memory with plain stores (ReduceScatter) instead of to
// every rank through the multicast alias (AllReduce).  U loads are in flight per lane.
template <bool kLocalDst, int U>
__device__ __forceinline__ void reduce_span_nvls(const char* mc_src, char* dst, long long n_vec,
                                                 int lane) {
  for (long long v0 = lane; v0 < n_vec; v0 += 32 * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (v0 + u * 32 < n_vec) v[u] = ptx::multimem_ld_reduce_bf16x8(mc_src + (v0 + u * 32) * 16);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (v0 + u * 32 < n_vec) {
        if (kLocalDst) ptx::st_global_v4(dst + (v0 + u * 32) * 16, v[u]);
        else ptx::multimem_st_v4(dst + (v0 + u * 32) * 16, v[u]);
      }
    }
  }
}

// AllReduce from slabs whose every 32-bit data word is followed by the epoch of the launch that
// wrote it (the producers' epilogues store them with 16-byte stores, so a data word and its
// epoch always arrive together): the reader needs no flag, no fence and no second round trip --
// it loads, and re-loads the vectors whose epoch words are not yet this launch's.  One output
// vector (8 bf16) = two slab vectors per source rank.  fp32 sum in rank order, deterministic.
template <int WT, int U>
__device__ __noinline__ bool reduce_span_ll(const char* const (&src)[kMaxWorld],
                                            char* const (&dst)[kMaxWorld], int W, int n_vec,
                                            uint32_t epoch, int lane, const WaitCtx& wc) {
  for (int v0 = lane; v0 < n_vec; v0 += 32 * U) {
    uint4 a[U][WT][2];
    // Load the whole batch, look at all epoch words, and re-load the whole batch while any of
    // them is not this launch's: the loads of a batch stay independent of one another, so a
    // retry costs one memory latency, not one per vector.
    uint32_t it = 0;
    uint64_t t0 = 0;
    while (true) {
      bool all = true;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long off = static_cast<long long>(v0 + u * 32) * 32;
        if (v0 + u * 32 < n_vec) {
#pragma unroll
          for (int c = 0; c < WT; ++c) {
            if (c < W) {
              a[u][c][0] = ptx::ld_relaxed_sys_v4(reinterpret_cast<const uint32_t*>(src[c] + off));
              a[u][c][1] = ptx::ld_relaxed_sys_v4(reinterpret_cast<const uint32_t*>(src[c] + off + 16));
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (v0 + u * 32 < n_vec) {
#pragma unroll
          for (int c = 0; c < WT; ++c) {
            if (c < W) {
#pragma unroll
              for (int h = 0; h < 2; ++h)
                all = all && a[u][c][h].y == epoch && a[u][c][h].w == epoch;
            }
          }
        }
      }
      if (all) break;
      // bounded: same budget and abort protocol as every other wait of the kernel
      ++it;
      if (it > 8) __nanosleep(it > 1024 ? 400 : 60);
      if ((it & 63u) == 0u) {
        bool give_up = *wc.s_abort != 0u ||
                       (wc.status != nullptr && ptx::ld_relaxed_sys(wc.status) != 0u);
        const uint64_t now = global_timer_ns();
        if (t0 == 0) t0 = now;
        else if (!give_up && now - t0 > wc.limit_ns) {
          report_failure(wc, ST_TIMEOUT_TILE, 0xFFu, static_cast<uint32_t>(v0));
          give_up = true;
        }
        if (give_up) { *wc.s_abort = 1u; return false; }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * 32;
      if (v >= n_vec) continue;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < WT; ++c) {
        if (c >= W) continue;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint4 x = a[u][c][h];
          acc[h * 4 + 0] += __uint_as_float(x.x << 16);
          acc[h * 4 + 1] += __uint_as_float(x.x & 0xffff0000u);
          acc[h * 4 + 2] += __uint_as_float(x.z << 16);
          acc[h * 4 + 3] += __uint_as_float(x.z & 0xffff0000u);
        }
      }
      uint4 r;
      r.x = ptx::pack_bf16x2(acc[0], acc[1]);
      r.y = ptx::pack_bf16x2(acc[2], acc[3]);
      r.z = ptx::pack_bf16x2(acc[4], acc[5]);
      r.w = ptx::pack_bf16x2(acc[6], acc[7]);
#pragma unroll
      for (int d = 0; d < WT; ++d)
        if (d < W && dst[d] != nullptr) ptx::st_global_v4(dst[d] + static_cast<long long>(v) * 16, r);
    }
  }
  return true;
}

// One exchange worker (a full warp).  Pulls items until the queue is empty.  Returns when done
// or when a wait expired.  `s_items_done` is the CTA's count of finished AllReduce items.
template <int OP, int R>
__device__ __forceinline__ void exchange_worker(const OpParams& p, uint32_t ring, WaitCtx& wc,
                                                uint32_t epoch, volatile uint32_t* s_items_done,
                                                volatile uint32_t* s_progress) {
  const Sched& s = p.sched;
  const int lane = threadIdx.x & 31;
  const int W = s.world;
  if (W <= 1 || p.n_items <= 0) return;
  wc.where = (blockIdx.x << 8) | 0x10u | (threadIdx.x >> 5);
  const bool nvls_ag = OP == OP_AG && p.use_nvls && p.mc_data != nullptr;
  // one item serves every receiver: through the multicast alias, or by storing to each peer
  const bool bcast_ag = nvls_ag || (OP == OP_AG && p.ag_fanout != 0);
  const bool nvls_ar = OP == OP_AR && p.use_nvls && !s.one_shot && p.mc_data != nullptr &&
                       p.mc_out != nullptr;
  const bool nvls_rs = OP == OP_RS && p.use_nvls && p.mc_data != nullptr;
  const long long row_bytes = (OP == OP_AG ? static_cast<long long>(p.K) : static_cast<long long>(s.N)) * 2;
  char* const local = static_cast<char*>(p.peer_data[s.rank]);
  uint32_t entered_mask = 1u << s.rank;  // ranks known to have entered this launch
  // Items normally come from a queue (an atomic counter), so that early items meet early data.
  // The latency-bound AllReduce over epoch-carrying slabs hands them out statically instead --
  // worker w takes items w, w + workers, ... -- which saves every worker the counter's round
  // trip to L2 before its first load (every warp of the grid is a worker there).
  const bool fixed_items = OP == OP_AR && s.ar_push == 2;
  const uint32_t n_workers = gridDim.x * (kThreads / 32);
  uint32_t next_item = 0;
  if (fixed_items) next_item = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  else if (lane == 0) next_item = atomicAdd(p.sync + SW_NEXT_ITEM, 1u);

  while (true) {
    // The queue is read one item ahead: the atomic for the next item is in flight while this
    // one is processed, so its round trip to L2 is off the critical path.
    const int item = static_cast<int>(__shfl_sync(0xffffffffu, next_item, 0));
    if (item >= p.n_items) break;
    if (fixed_items) next_item += n_workers;
    else if (lane == 0) next_item = atomicAdd(p.sync + SW_NEXT_ITEM, 1u);

    if (OP == OP_AG) {
      // Item order: row-block j of the own shard goes to every receiver (nearest ring distance
      // first) before row-block j+1 goes to anybody -- the order in which receivers consume.
      // K-range form (ag_cv_log2 != 0): range g of row-block j goes to every receiver before
      // range g + 1 goes to anybody, so all receivers can start on the row-block early.
      const int lg_cv = p.ag_cv_log2;
      const int per_block = (bcast_ag ? 1 : W - 1) * kGatherSub;
      const int j = item / per_block;
      const int in_block = item % per_block;
      // receiver's ring distance, and the 4-row group or K-range
      const int d = bcast_ag ? 0 : 1 + (lg_cv != 0 ? in_block % (W - 1) : in_block / kGatherSub);
      const int g = lg_cv != 0 ? in_block / (W - 1) : in_block % kGatherSub;
      const int rowblock = s.rank * s.part_blocks + j;
      const int rows_in_block = rowblock_rows(s, rowblock);
      const int r0 = g * (kBlockM / kGatherSub);
      int r1 = r0 + kBlockM / kGatherSub;
      if (r1 > rows_in_block) r1 = rows_in_block;
      const int n_vec = r1 > r0 ? static_cast<int>((r1 - r0) * row_bytes / 16) : 0;
      const long long base = (static_cast<long long>(rowblock_row0(s, rowblock)) + r0) * row_bytes;
      const int dst_rank = (s.rank - d + W) % W;
      char* dst = nvls_ag ? static_cast<char*>(p.mc_data) : static_cast<char*>(p.peer_data[dst_rank]);
      // The receiver's gathered buffer may be overwritten only once the receiver has entered
      // this launch (its previous launch, which read the buffer, has ended).
      {
        const int first = bcast_ag ? 0 : dst_rank, last = bcast_ag ? W - 1 : dst_rank;
        bool ok = true;
        for (int r = first + lane; r <= last && ok; r += 32) {
          if (entered_mask & (1u << r)) continue;
          const uint32_t* f = p.sync + SW_ENTRY + r;
          ok = bounded_wait<true>(wc, [&] { return reached(ptx::ld_acquire_sys(f), epoch); },
                                  ST_TIMEOUT_ENTRY, r, epoch);
        }
        if (!__all_sync(0xffffffffu, ok)) return;
        for (int r = first; r <= last; ++r) entered_mask |= 1u << r;
      }
      if (p.ag_lead_tiles > 0 && s_progress != nullptr) {
        // Pacing: rows pushed long before their consumers need them only compete with the GEMM
        // (here and at the receiver) for memory bandwidth and cache.  The receivers walk the same
        // raster as this rank, so this CTA's own progress stands in for theirs: wait until the
        // GEMM is within ag_lead_tiles of the raster group that consumes these rows.
        const int pos = s.part_blocks + j * (W - 1) + (bcast_ag ? 0 : d - 1);
        const int need = (pos / s.group_rows) * s.group_rows * s.Q - p.ag_lead_tiles;
        if (need > 0) {
          const bool ok = bounded_wait<true>(
              wc, [&] { return static_cast<int>(*s_progress) >= need; }, ST_TIMEOUT_PACE, item, need);
          if (!__all_sync(0xffffffffu, ok)) return;
        }
      }
      if (lg_cv != 0) {
        const int first_vec = g << lg_cv;
        const int row_vecs = static_cast<int>(row_bytes / 16);
        int valid_cv = row_vecs - first_vec;
        if (valid_cv > (1 << lg_cv)) valid_cv = 1 << lg_cv;
        const long long cbase = static_cast<long long>(rowblock_row0(s, rowblock)) * row_bytes +
                                static_cast<long long>(first_vec) * 16;
        if (!diag(p, 1) && valid_cv > 0 && rows_in_block > 0)
          push_chunk<R>(local + cbase, dst + cbase, rows_in_block, row_bytes, lg_cv, valid_cv, ring,
                        lane);
      } else if (!diag(p, 1)) {
        if (bcast_ag && !nvls_ag) {
          char* fan[kMaxWorld - 1];
#pragma unroll
          for (int i = 0; i < kMaxWorld - 1; ++i)
            fan[i] = i < W - 1 ? static_cast<char*>(p.peer_data[(s.rank - 1 - i + W) % W]) + base
                               : nullptr;
          push_span<R, kMaxWorld - 1>(local + base, fan, W - 1, n_vec, false, ring, lane,
                                      kDiag ? p.debug_flags : 0);
        } else if (p.push_bulk && !nvls_ag) {
          push_span_bulk<R>(local + base, dst + base, n_vec, ring, lane);
        } else {
          char* one[1] = {dst + base};
          push_span<R, 1>(local + base, one, 1, n_vec, nvls_ag, ring, lane,
                          kDiag ? p.debug_flags : 0);
        }
      }
      __syncwarp();
      if (lane == 0) {
        ptx::fence_acq_rel_sys();
        const long long idx = SW_FLAGS + gather_flag_index(rowblock, g);
        if (bcast_ag) {
          for (int i = 1; i < W; ++i)
            ptx::st_relaxed_sys(p.peer_sync[(s.rank - i + W) % W] + idx, epoch);
        } else {
          ptx::st_relaxed_sys(p.peer_sync[dst_rank] + idx, epoch);
        }
      }
    } else {
      const int cpb = reduce_chunks_per_piece(s, p.item_vecs);
      const int k = item / cpb, c = item % cpb;
      const int rb = owner_first_block(s, s.rank) + k;
      const bool ll = OP == OP_AR && s.ar_push == 2;   // slabs carry their own epochs: no flags
      // 1. the row-block is complete once every rank has published every column block of it
      uint32_t* summary = p.sync + SW_FLAGS + summary_flag_index(s, rb);
      bool ready = ll || ptx::ld_acquire_gpu(summary) == epoch;
      ready = __shfl_sync(0xffffffffu, ready, 0);
      if (!ready && c != 0) {
        // Only the worker holding the first chunk of a piece polls the W x Q tile flags (items
        // are handed out in order, so somebody always holds it); everybody else waits for the
        // one summary word instead of hammering the lines the peers are writing to.
        const bool ok = bounded_wait<true>(wc, [&] { return ptx::ld_acquire_gpu(summary) == epoch; },
                                           ST_TIMEOUT_TILE, rb, 1);
        if (!__all_sync(0xffffffffu, ok)) return;
      } else if (!ready) {
        bool ok = true;
        if ((s.Q & 3) == 0) {
          // The Q flags of one source rank are contiguous: poll them four at a time, all of a
          // lane's vectors per round (independent loads, one memory latency per round).
          const int vq = s.Q >> 2, n_v = W * vq;
          ok = bounded_wait<true>(wc, [&] {
            bool all = true;
            for (int idx = lane; idx < n_v; idx += 32) {
              const int src = idx / vq, q4 = idx % vq;
              const uint4 v = ptx::ld_relaxed_sys_v4(p.sync + SW_FLAGS +
                                                     tile_flag_index(s, src, rb, q4 * 4));
              all = all && v.x == epoch && v.y == epoch && v.z == epoch && v.w == epoch;
            }
            return all;
          }, ST_TIMEOUT_TILE, rb, 0);
          ptx::fence_acq_rel_sys();
        } else {
          for (int idx = lane; idx < W * s.Q && ok; idx += 32) {
            const int src = idx / s.Q, q = idx % s.Q;
            const uint32_t* f = p.sync + SW_FLAGS + tile_flag_index(s, src, rb, q);
            ok = bounded_wait<true>(wc, [&] { return ptx::ld_acquire_sys(f) == epoch; },
                                    ST_TIMEOUT_TILE, (src << 24) | rb, q);
          }
        }
        if (!__all_sync(0xffffffffu, ok)) return;
        if (lane == 0) stamp(p, 2);
        if (lane == 0) ptx::st_release_gpu(summary, epoch);
      }
      // 2. sum this chunk of the piece
      int row0, row1;
      owner_item_rows(s, s.rank, k, &row0, &row1);
      const long long piece_vecs = static_cast<long long>(row1 - row0) * row_bytes / 16;
      const long long v_begin = static_cast<long long>(c) * p.item_vecs;
      long long n_vec = piece_vecs - v_begin;
      if (n_vec > p.item_vecs) n_vec = p.item_vecs;
      if (n_vec > 0 && !diag(p, 1)) {
        const long long base = static_cast<long long>(row0) * row_bytes + v_begin * 16;
        if (nvls_ar) {
          reduce_span_nvls<false, 8>(static_cast<const char*>(p.mc_data) + base,
                                     static_cast<char*>(p.mc_out) + base, n_vec, lane);
        } else if (nvls_rs) {
          // every rank's partial of these rows sits at the same offset of its own buffer
          reduce_span_nvls<true, 16>(static_cast<const char*>(p.mc_data) + base, local + base, n_vec,
                                     lane);
        } else if (ll) {
          const char* src[kMaxWorld];
          char* dst[kMaxWorld];
#pragma unroll
          for (int r = 0; r < kMaxWorld; ++r) {
            src[r] = r >= W ? nullptr
                            : reinterpret_cast<const char*>(p.sync) + kArSlabByteOffset +
                                  ((static_cast<long long>(r) * s.part_rows + (row0 - s.rank * s.part_rows)) *
                                       row_bytes + v_begin * 16) * 2;
            dst[r] = r >= W ? nullptr : static_cast<char*>(p.peer_out[r]) + base;
          }
          bool ok;
          if (W <= 2) ok = reduce_span_ll<2, 4>(src, dst, W, static_cast<int>(n_vec), epoch, lane, wc);
          else if (W <= 4) ok = reduce_span_ll<4, 2>(src, dst, W, static_cast<int>(n_vec), epoch, lane, wc);
          else ok = reduce_span_ll<8, 1>(src, dst, W, static_cast<int>(n_vec), epoch, lane, wc);
          if (!__all_sync(0xffffffffu, ok)) return;
          if (item == 0 && lane == 0) stamp(p, 2);
        } else {
          ReduceSpan sp;
          sp.n_vec = static_cast<int>(n_vec);
          sp.mc_dst = (OP == OP_AR && p.use_nvls && !s.one_shot && p.mc_out != nullptr)
                          ? static_cast<char*>(p.mc_out) + base : nullptr;
#pragma unroll
          for (int r = 0; r < kMaxWorld; ++r) {
            // RS: slab r of this rank's buffer holds rank r's partial of this rank's rows.
            // AR with staging slabs: slab r of this rank's barrier buffer, same rows.
            sp.src[r] = r >= W ? nullptr
                        : (OP == OP_RS)
                            ? local + base + (static_cast<long long>(r) - s.rank) * s.part_rows * row_bytes
                        : (OP == OP_AR && s.ar_push)
                            ? reinterpret_cast<const char*>(p.sync) + kArSlabByteOffset +
                                  (static_cast<long long>(r) * s.part_rows + (row0 - s.rank * s.part_rows)) * row_bytes +
                                  v_begin * 16
                            : static_cast<const char*>(p.peer_data[r]) + base;
            sp.dst[r] = r >= W ? nullptr
                        : (OP == OP_RS) ? local + base : static_cast<char*>(p.peer_out[r]) + base;
            // one-shot AllReduce: every rank reduces every row, for its own output only
            if (OP == OP_AR && s.one_shot && r < W && r != s.rank) sp.dst[r] = nullptr;
          }
          if (W <= 2) reduce_span<OP, 2, R>(sp, W, ring, lane);
          else if (W <= 4) reduce_span<OP, 4, R>(sp, W, ring, lane);
          else reduce_span<OP, 8, R>(sp, W, ring, lane);
        }
      }
      __syncwarp();
    }

    // 3. AllReduce: count the item.  Its results went to other GPUs with plain stores; they are
    //    made visible, and the rank's completion is announced, once per CTA at teardown (a
    //    system-scope fence per item would serialise the warps of an SM behind one another).
    if (OP == OP_AR && lane == 0) {
      atomicAdd(const_cast<uint32_t*>(s_items_done), 1u);
      stamp_max(p, 6);
    }
    __syncwarp();
  }
}

// AllReduce, once per CTA after all of its warps have finished: publish the results of the items
// this CTA reduced, add them to the rank's count, and when that completes the rank's items tell
// every rank that this rank has written its share of their outputs and reads no more partials.
__device__ __forceinline__ void announce_reduced_items(const OpParams& p, uint32_t n_done,
                                                       uint32_t epoch) {
  if (n_done == 0u) return;
  ptx::fence_acq_rel_sys();
  const uint32_t before = atomicAdd(p.sync + SW_ITEMS_DONE, n_done);
  if (before + n_done == static_cast<uint32_t>(p.n_items)) {
    stamp(p, 3);
    for (int r = 0; r < p.sched.world; ++r)
      ptx::st_relaxed_sys(p.peer_sync[r] + SW_EXIT + p.sched.rank, epoch);
  }
}

// ------------------------------------------------------------------------------------------
// Kernel
// ------------------------------------------------------------------------------------------
template <int OP, int CG>
__global__ void __launch_bounds__(kThreads, 1)
fused_gemm_kernel(const __grid_constant__ CUtensorMap tma_a,
                  const __grid_constant__ CUtensorMap tma_b,
                  const __grid_constant__ OpParams p) {
  extern __shared__ uint8_t smem_raw[];
  const Sched& s = p.sched;
  const int warp = threadIdx.x >> 5;
  // Shared-memory layout (1024-byte aligned): [barriers + control words, 1 KB][operand stages]
  // [epilogue transpose buffers, 16 KB][ring of the in-CTA exchange warp].  The control block
  // comes first so that no ring -- in particular the 160 KB of rings of a dedicated exchange
  // CTA, which reuse the stage region and whatever follows it -- can ever overlap it.
  const uint32_t smem_aligned = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_aligned;
  const uint32_t smem_base = smem_aligned + kSmemBarrierBytes;          // operand stages
  const int ring_bytes = p.stages * stage_bytes_cg(s.block_n, CG);
  const uint32_t epi_stage = smem_base + ring_bytes;
  const uint32_t xchg_ring = epi_stage + kEpilogueStageBytes;
  uint8_t* gen_base = smem_raw + (smem_aligned - ptx::smem_u32(smem_raw));
  volatile uint32_t* s_words = reinterpret_cast<volatile uint32_t*>(gen_base + 8 * BAR_COUNT);
  volatile uint32_t* s_tmem = s_words;       // TMEM base address
  volatile uint32_t* s_abort = s_words + 1;  // CTA-wide abort flag
  volatile uint32_t* s_epoch = s_words + 2;
  volatile uint32_t* s_progress = s_words + 3;  // AllGather: tile the TMA producer has reached
  volatile uint32_t* s_items_done = s_words + 4;  // AllReduce: items this CTA's warps reduced
  const bool is_comm = static_cast<int>(blockIdx.x) < p.n_comm;

  const bool tr = kDiag && p.trace != nullptr;   // coarse counters
  const long long tr_c0 = diag_clock(tr);
  const uint64_t tr_t0 = tr ? global_timer_ns() : 0;

  WaitCtx wc;
  wc.status = p.status;
  wc.s_abort = s_abort;
  wc.limit_ns = p.wait_limit_ns;
  wc.where = blockIdx.x << 8;

  if (threadIdx.x == 0) {
    *s_abort = 0u;
    *s_progress = 0u;
    *s_items_done = 0u;
    s_words[5] = 0u;            // epilogue warps that have stored their rows of a tail piece
    s_words[6] = 0u;            // set once s_epoch holds this launch's epoch
    if (!is_comm) {
      for (int i = 0; i < kMaxStages; ++i) {
        ptx::mbar_init(bar_base + 8u * (BAR_FULL + i), 1);
        ptx::mbar_init(bar_base + 8u * (BAR_EMPTY + i), 1);
      }
      const bool publishes = (OP == OP_RS || OP == OP_AR) && s.world > 1;
      for (int i = 0; i < 2; ++i) {
        ptx::mbar_init(bar_base + 8u * (BAR_TFULL + i), 1);
        // accumulator free again: 4 epilogue warps (+ the publisher) of every CTA sharing it
        ptx::mbar_init(bar_base + 8u * (BAR_TEMPTY + i), (publishes ? 5 : 4) * CG);
        ptx::mbar_init(bar_base + 8u * (BAR_STORED + i), 4);
      }
      ptx::tma_prefetch_desc(&tma_a);
      ptx::tma_prefetch_desc(&tma_b);
    }
    ptx::fence_mbar_init();
  }
  if (CG == 2 && !is_comm) ptx::cluster_sync_all();  // both CTAs' barriers exist before any use
  if (!is_comm && warp == 1) {
    if (CG == 1) {
      ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(s_tmem)), 512);
      ptx::tmem_relinquish();
    } else {
      ptx::tmem_alloc_pair(ptx::smem_u32(const_cast<uint32_t*>(s_tmem)), 512);
      ptx::tmem_relinquish_pair();
    }
  }
  // Everything above touched only this CTA's shared and tensor memory, so with a programmatic
  // dependent launch it overlaps the tail of the previous kernel in the stream.  From here on
  // global memory is read (epoch, flags, operands the previous kernel may have produced): wait
  // for the previous kernel to complete, then let the NEXT kernel's CTAs start their own set-up
  // as SMs become free (they stop at the same wait until this kernel has completed).
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();
  ptx::tc_fence_before();
  __syncthreads();            // barriers initialised, tensor-memory address published
  ptx::tc_fence_after();
  // The launch epoch lives on the device (graph replays need no host state) unless the caller
  // supplies one (GEMM+AR and the multi-node style signatures pass a host epoch).  Reading it is
  // a round trip to memory, so it is kept off the path of the warps that start the GEMM: lane 0
  // of the exchange warp reads it, and only the warps that use it (publisher, exchange and
  // epilogue warps; everybody in an exchange CTA and in AllGather, whose TMA producer compares
  // arrival flags with it) meet at a named barrier; the TMA producer and the MMA issuer of the
  // other operators run on.
  uint32_t epoch = p.epoch_arg;
  if (p.sync != nullptr) {
    const bool all_meet = is_comm || OP == OP_AG;
    if (threadIdx.x == 96) {
      uint32_t e = p.epoch_arg;
      if (e == 0u) e = ptx::ld_relaxed_sys(p.sync + SW_EPOCH) + 1u;
      *s_epoch = e;
      __threadfence_block();
      s_words[6] = 1u;          // for the warps that do not meet at the barrier below
      if (blockIdx.x == 0) stamp(p, 0);
      if (blockIdx.x == 0 && s.world > 1) {
        // AG / RS: tell every rank that this rank has entered launch e, i.e. that its previous
        // launch has ended and its buffers may be written again (replaces an all-rank barrier).
        if (OP == OP_AG || OP == OP_RS)
          for (int r = 0; r < s.world; ++r) ptx::st_release_sys(p.peer_sync[r] + SW_ENTRY + s.rank, e);
        // AR: a rank with nothing to reduce still owes its peers the "finished" signal.
        if (OP == OP_AR && p.n_items <= 0)
          for (int r = 0; r < s.world; ++r) ptx::st_release_sys(p.peer_sync[r] + SW_EXIT + s.rank, e);
      }
    }
    if (all_meet) {
      ptx::named_barrier_sync(1, kThreads);
      epoch = *s_epoch;
    } else if (warp >= 2) {
      ptx::named_barrier_sync(1, kThreads - 64);
      epoch = *s_epoch;
    }
  }

  if (is_comm) {
    if (OP != OP_GEMM)
      exchange_worker<OP, kRingDedicated>(p, smem_base + warp * (kRingDedicated * 32 * 16), wc,
                                          epoch, s_items_done, nullptr);
  } else if (warp == 3) {
    if (OP == OP_AR && s.ar_push == 2 && s.world > 1) {
      wc.where = (blockIdx.x << 8) | 3u;
      const bool ok = bounded_wait<true>(wc, [&] { return *s_progress != 0u; }, ST_TIMEOUT_PIPE,
                                         0x600u, 0u);
      (void)ok;   // on expiry the abort flag is up and the worker returns at its first wait
    }
    if (OP != OP_GEMM) {
      if (p.ring_slots == kRingInCtaDeep)
        exchange_worker<OP, kRingInCtaDeep>(p, xchg_ring, wc, epoch, s_items_done, s_progress);
      else
        exchange_worker<OP, kRingInCta>(p, xchg_ring, wc, epoch, s_items_done, s_progress);
    }
  } else {
    compute_roles<OP, CG>(&tma_a, &tma_b, p, smem_base, bar_base, epi_stage, *s_tmem, wc, epoch,
                          s_progress);
    // Latency-bound AllReduce over epoch-carrying slabs: its reduce items need no shared-memory
    // ring, so every warp whose GEMM role has ended joins the exchange worker on the item queue.
    if (OP == OP_AR && s.ar_push == 2 && s.world > 1) {
      __syncwarp();
      if (warp < 2) {
        // the TMA producer and the MMA issuer skipped the epoch barrier: pick the epoch up now
        const bool ok = bounded_wait<true>(wc, [&] { return s_words[6] != 0u; }, ST_TIMEOUT_PIPE,
                                           0x700u, 0u);
        (void)ok;   // on expiry the abort flag is up and the worker returns at its first wait
        __threadfence_block();
        epoch = *s_epoch;
      }
      exchange_worker<OP, kRingInCta>(p, xchg_ring, wc, epoch, s_items_done, nullptr);
    }
  }

  // ---------------- teardown ----------------
  if (*s_abort != 0u) {
    // Leave time for copies this CTA still has in flight to land before its shared memory and
    // tensor memory are released.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 50000ull) __nanosleep(1000);
  }
  ptx::tc_fence_before();
  __syncthreads();
  // A pair leaves together: the peer may still signal this CTA's barriers or read its operands.
  if (CG == 2 && !is_comm) ptx::cluster_sync_all();
  if (!is_comm && warp == 1) {
    __syncwarp();
    ptx::tc_fence_after();
    if (CG == 1) ptx::tmem_dealloc(*s_tmem, 512);
    else ptx::tmem_dealloc_pair(*s_tmem, 512);
  }
  if (tr && threadIdx.x == 0) {
    p.trace[blockIdx.x * 16 + 0] = clock64() - tr_c0;
    p.trace[blockIdx.x * 16 + 1] = global_timer_ns() - tr_t0;
  }
  if (p.sync == nullptr || threadIdx.x != 96) return;   // the thread that holds the epoch
  // AllReduce over epoch-carrying slabs: items are assigned statically and every CTA passes
  // here when its warps have finished theirs, so "this rank has finished its exchange work" is
  // the moment the last CTA arrives below -- no separate item count.  The reduced rows went into
  // the peers' outputs with plain stores, so every CTA still makes its own stores visible
  // system-wide before it is counted.  The other forms publish through announce_reduced_items.
  const bool ll_exit = OP == OP_AR && s.world > 1 && s.ar_push == 2;
  if (OP == OP_AR && s.world > 1 && !ll_exit && *s_abort == 0u)
    announce_reduced_items(p, *s_items_done, epoch);

  // ---------------- exit handshake (one thread of every CTA) ----------------
  wc.where = (blockIdx.x << 8) | 15u;
  if (ll_exit) ptx::fence_acq_rel_sys();
  else __threadfence();
  // A CTA that gave up on a wait marks the count, so that the last one does not report the
  // rank's exchange work as finished.
  const uint32_t arrive = *s_abort == 0u ? 1u : 0x10001u;
  const uint32_t done = atomicAdd(p.sync + SW_GRID_DONE, arrive);
  if ((done & 0xffffu) == gridDim.x - 1) {
    // Last CTA of this rank.  AllReduce: the kernel may only end when every rank has finished
    // its exchange work (this rank's output is complete, nobody still reads its partials).
    // AG / RS need no such wait: their results are produced by this rank's own CTAs, and the
    // next launch's writers wait for the entry flag instead.
    stamp(p, 4);
    const bool clean = ((done + arrive) >> 16) == 0u;
    if (ll_exit && clean && p.n_items > 0) {
      for (int r = 0; r < s.world; ++r)
        ptx::st_relaxed_sys(p.peer_sync[r] + SW_EXIT + s.rank, epoch);
    }
    if (OP == OP_AR && s.world > 1 && *s_abort == 0u) {
      for (int r = 0; r < s.world; ++r) {
        const uint32_t* f = p.sync + SW_EXIT + r;
        if (!bounded_wait<true>(wc, [&] { return reached(ptx::ld_acquire_sys(f), epoch); },
                                ST_TIMEOUT_EXIT, r, epoch))
          break;
      }
    }
    stamp(p, 5);
    // Plain stores: the end of the kernel makes them visible to the next launch.
    p.sync[SW_GRID_DONE] = 0u;
    p.sync[SW_NEXT_ITEM] = 0u;
    p.sync[SW_ITEMS_DONE] = 0u;
    p.sync[SW_EPOCH] = epoch;
  }
}

}  // namespace mkb
