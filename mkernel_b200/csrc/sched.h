// Tile scheduling and synchronisation-word layout shared by host and device code.
//
// All three fused operators run the same persistent bf16 GEMM over output tiles of
// 128 rows x block_n columns.  What differs is (1) the order in which row-blocks are visited,
// chosen so that the exchange step has work as early as possible, and (2) which flags a tile
// waits for or raises.  Everything in this header is plain integer arithmetic so that the
// same functions can be unit-tested on the host through the C ABI (mk_sched_* functions).
//
// Reference behaviour restated here (not its code): AllGather+GEMM visits the local shard first
// and then the shards at ring distance 1..W-1 (src/ag_gemm_warp_specialized.cu:243; here the
// remote shards are interleaved by row-block to match the order in which pushes arrive); the
// reduce-scatter family interleaves the owners' slices so every owner's tiles become complete
// progressively (include/operators/gemm_rs/gemm_rs.cuh:279-353).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define MKB_HD __host__ __device__ __forceinline__
#else
#define MKB_HD inline
#endif

namespace mkb {

constexpr int kMaxWorld = 8;
constexpr int kBlockM = 128;
constexpr int kBlockK = 64;
constexpr int kThreads = 256;
constexpr int kGatherSub = 32;         // AllGather: a 128-row block lands as 32 groups of 4 rows
constexpr int kRingDedicated = 40;     // 16-byte ring slots per lane, warps of an exchange CTA
constexpr int kRingInCta = 32;         // same for the exchange warp inside a compute CTA (16 KB)
constexpr int kEpilogueStageBytes = 16384;  // 4 epilogue warps x 32 rows x 128 B transpose buffers
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 232448;    // 227 KiB opt-in limit per CTA on sm_100
constexpr int kSmemBarrierBytes = 1024;  // barriers + control words, FIRST in shared memory

enum OpKind : int { OP_GEMM = 0, OP_AG = 1, OP_RS = 2, OP_AR = 3 };

// Word offsets inside an operator's synchronisation buffer (uint32 words, caller-owned,
// symmetric across ranks, zeroed once before first use).
enum SyncWord : int {
  SW_ENTRY = 0,       // [0,8): slot per rank: "rank s has entered launch <epoch>" (AG, RS)
  SW_EPOCH = 8,       // device-resident epoch of the last finished launch (AG, RS)
  SW_GRID_DONE = 9,   // CTAs that reached the end of the kernel in the low 16 bits, CTAs that
                      // gave up on a wait above them (reset by the last CTA)
  SW_NEXT_ITEM = 10,  // next exchange work item to hand out (reset by the last CTA)
  SW_ITEMS_DONE = 11, // exchange work items completed, for the AllReduce forms that hand items
                      // out through the queue (reset by the last CTA)
  SW_STATUS = 12,     // [12,16): {code, where, detail0, detail1}; 0 = healthy
  SW_EXIT = 16,       // [16,24): exit slot per rank: "rank s finished its exchange work" (AR)
  SW_FLAGS = 64,      // per-tile / per-row-group flags start here
};

// Status codes written to SW_STATUS (first failure wins).
enum StatusCode : int {
  ST_OK = 0,
  ST_TIMEOUT_PIPE = 1,      // intra-CTA mbarrier wait expired
  ST_TIMEOUT_GATHER = 2,    // AllGather: gathered-rows flag never arrived
  ST_TIMEOUT_TILE = 3,      // reduce role: a peer's tile flag never arrived
  ST_TIMEOUT_EXIT = 4,      // exit handshake: a peer never reported completion
  ST_TIMEOUT_ENTRY = 5,     // entry barrier (prepare): a peer never arrived
  ST_TIMEOUT_COPY = 6,      // exchange role: a bulk copy never completed
  ST_TIMEOUT_PACE = 7,      // AllGather push pacing: this CTA's GEMM never reached the tile
};

struct Sched {
  int op;          // OpKind
  int rank, world;
  int M, N;        // rows / cols of this rank's GEMM output
  int block_n;
  int part_rows;   // AG: rows per gathered shard; RS/AR: rows per owner; GEMM: M
  int part_blocks; // ceil(part_rows / 128)
  int P;           // row-blocks: AG: world*part_blocks, else ceil(M/128)
  int Q;           // column blocks: ceil(N / block_n)
  int group_rows;  // raster group height in row-blocks
  int group_cols;  // raster group width in column blocks (Q = the whole width)
  int interleave;  // RS/AR: 1 when part_rows % 128 == 0 (owner-interleaved order)
  int one_shot;    // AR only: every rank reduces every row for itself (no result broadcast)
  int ar_push;     // AR only: partial rows are also stored into their owner's staging slabs (in
                   // the upper half of the barrier buffer), so owners reduce from local memory.
                   // 1: plain slabs + tile flags; 2: slabs whose data words carry the epoch
};

MKB_HD int ceil_div(int a, int b) { return (a + b - 1) / b; }

MKB_HD Sched make_sched(int op, int rank, int world, int M, int N, int block_n, int group_rows,
                        int group_cols = 0) {
  Sched s;
  s.op = op; s.rank = rank; s.world = world; s.M = M; s.N = N; s.block_n = block_n;
  if (op == OP_AG) s.part_rows = M / world;              // rows of one gathered shard
  else if (op == OP_GEMM || world == 1) s.part_rows = M;
  else s.part_rows = ceil_div(M, world);                 // rows reduced by one owner
  if (s.part_rows < 1) s.part_rows = 1;
  s.part_blocks = ceil_div(s.part_rows, kBlockM);
  s.P = (op == OP_AG) ? world * s.part_blocks : ceil_div(M, kBlockM);
  s.Q = ceil_div(N, block_n);
  s.group_rows = group_rows < 1 ? 1 : group_rows;
  // Column grouping makes a second pass over all rows, which the row-ordered exchanges (rows
  // consumed as they arrive, owners served round by round) cannot afford: one GPU only.
  s.group_cols = (group_cols < 1 || group_cols > s.Q || world > 1) ? s.Q : group_cols;
  s.interleave = ((op == OP_RS || op == OP_AR) && world > 1 && (s.part_rows % kBlockM) == 0 &&
                  s.part_blocks * world == s.P) ? 1 : 0;
  s.one_shot = 0;
  s.ar_push = 0;
  return s;
}

// i-th row-block in visiting order -> row-block id.
//   AG: id = shard * part_blocks + j; the local shard first, then the remote shards
//   row-block-major (block j of ring distance 1..W-1, then block j+1, ...).
//   RS/AR (interleaved): j-th block of owner (rank+1+d) % W, d fastest, so the own slice is last
//   inside each round and every owner receives complete row-blocks round by round.
MKB_HD int order_to_rowblock(const Sched& s, int i) {
  if (s.op == OP_AG) {
    // local shard first; then block j of every remote shard (ring distance 1..W-1) before block
    // j+1 of any: the senders push block j of their shard to everybody before block j+1, so
    // rows are consumed in the order in which they arrive
    if (i < s.part_blocks || s.world == 1) return s.rank * s.part_blocks + i;
    const int idx = i - s.part_blocks;
    const int j = idx / (s.world - 1), d = 1 + idx % (s.world - 1);
    return ((s.rank + d) % s.world) * s.part_blocks + j;
  }
  if (s.interleave) {
    const int j = i / s.world, d = i % s.world;
    return ((s.rank + 1 + d) % s.world) * s.part_blocks + j;
  }
  return i;
}

// Linear tile index -> (row-block id, column block).  Tiles are rastered in groups of
// group_rows row-blocks; inside a group the row-block index runs fastest so the CTAs working at
// the same time share a few A row-blocks and a contiguous range of B column blocks in L2.
// With group_cols < Q the raster is two-level: column groups outermost (all rows pass once per
// column group, so a group's slice of B plus one row group of A is what L2 has to hold).
MKB_HD void tile_to_coord(const Sched& s, int t, int* rowblock, int* q) {
  const int cg = t / (s.P * s.group_cols);            // full column groups precede a partial one
  const int q0 = cg * s.group_cols;
  const int cols_here = (s.Q - q0) < s.group_cols ? (s.Q - q0) : s.group_cols;
  const int tt = t - cg * s.P * s.group_cols;
  const int per_group = s.group_rows * cols_here;
  const int g = tt / per_group, r = tt % per_group;
  const int first = g * s.group_rows;
  const int rows_here = (s.P - first) < s.group_rows ? (s.P - first) : s.group_rows;
  const int i = first + r % rows_here;
  *q = q0 + r / rows_here;
  *rowblock = order_to_rowblock(s, i);
}

MKB_HD int rowblock_row0(const Sched& s, int rb) {
  if (s.op == OP_AG) return (rb / s.part_blocks) * s.part_rows + (rb % s.part_blocks) * kBlockM;
  return rb * kBlockM;
}
MKB_HD int rowblock_rows(const Sched& s, int rb) {
  if (s.op == OP_AG) {
    const int left = s.part_rows - (rb % s.part_blocks) * kBlockM;
    return left < kBlockM ? left : kBlockM;
  }
  const int left = s.M - rb * kBlockM;
  return left < kBlockM ? left : kBlockM;
}
MKB_HD int rowblock_shard(const Sched& s, int rb) { return rb / s.part_blocks; }  // AG only

// RS/AR: owners whose row range [o*part_rows, (o+1)*part_rows) intersects row-block rb.
MKB_HD void rowblock_owners(const Sched& s, int rb, int* lo, int* hi) {
  if (s.one_shot) { *lo = 0; *hi = s.world - 1; return; }
  const int r0 = rb * kBlockM;
  int r1 = r0 + kBlockM; if (r1 > s.M) r1 = s.M;
  *lo = r0 / s.part_rows;
  int h = (r1 - 1) / s.part_rows; if (h > s.world - 1) h = s.world - 1;
  *hi = h;
}

// RS/AR reduce items of owner `o`: item k is the intersection of the owner's rows with
// row-block (first_block + k).
MKB_HD int owner_first_block(const Sched& s, int o) {
  return s.one_shot ? 0 : (o * s.part_rows) / kBlockM;
}
MKB_HD int owner_num_items(const Sched& s, int o) {
  if (s.one_shot) return s.P;
  int r0 = o * s.part_rows, r1 = r0 + s.part_rows;
  if (r1 > s.M) r1 = s.M;
  if (r1 <= r0) return 0;
  return (r1 - 1) / kBlockM - r0 / kBlockM + 1;
}
MKB_HD void owner_item_rows(const Sched& s, int o, int k, int* row0, int* row1) {
  const int rb = owner_first_block(s, o) + k;
  int a = rb * kBlockM, b = a + kBlockM;
  if (s.one_shot) { *row0 = a; *row1 = b > s.M ? s.M : b; return; }
  const int r0 = o * s.part_rows;
  int r1 = r0 + s.part_rows; if (r1 > s.M) r1 = s.M;
  if (a < r0) a = r0;
  if (b > r1) b = r1;
  *row0 = a; *row1 = b;
}

// GEMM+AllReduce staging slabs: the reference's barrier buffer is 8 MiB (2 x 1024 x 1024 words)
// and the flags of a latency-bound shape need a few KiB of it; the upper 4 MiB hold, on every
// rank o, W slabs [part_rows][N] bf16: slab s = rank s's partial of o's rows.
constexpr long long kArSlabByteOffset = 4ll << 20;
constexpr long long kArSlabBytes = 4ll << 20;
// `mode` 1: plain bf16 slabs plus per-tile flags; 2: every data word followed by the epoch (twice
// the bytes, no flags).
MKB_HD bool ar_push_fits(const Sched& s, long long sync_bytes, int mode) {
  return s.op == OP_AR && s.world > 1 && !s.one_shot &&
         sync_bytes >= kArSlabByteOffset + kArSlabBytes &&
         (long long)s.world * s.part_rows * s.N * 2 * mode <= kArSlabBytes;
}

// Flag indices (relative to SW_FLAGS).
MKB_HD long long tile_flag_index(const Sched& s, int src, int rb, int q) {
  return ((long long)src * s.P + rb) * s.Q + q;
}
MKB_HD long long gather_flag_index(int rb, int sub) { return (long long)rb * kGatherSub + sub; }
MKB_HD long long sync_words_needed(const Sched& s) {
  if (s.op == OP_AG) return SW_FLAGS + (long long)s.P * kGatherSub;
  // per-tile flags of every source rank, then one "row-block complete" summary word per block
  if (s.op == OP_RS || s.op == OP_AR) return SW_FLAGS + (long long)s.world * s.P * s.Q + s.P;
  return SW_FLAGS;
}
MKB_HD long long summary_flag_index(const Sched& s, int rb) {
  return (long long)s.world * s.P * s.Q + rb;
}

// Exchange work items.  AllGather: one item = one 16-row group of the own shard for one
// receiving rank (peer-major, nearest deadline first) or, through NVSwitch multicast, for all
// ranks at once.  ReduceScatter / AllReduce: the rows an owner reduces, cut at row-block
// boundaries into pieces and every piece into chunks of item_vecs 16-byte vectors.
MKB_HD int gather_num_items(const Sched& s, int nvls) {
  return (nvls ? 1 : s.world - 1) * s.part_blocks * kGatherSub;
}
MKB_HD int reduce_chunks_per_piece(const Sched& s, int item_vecs) {
  int rows = (s.part_rows < kBlockM && !s.one_shot) ? s.part_rows : kBlockM;
  long long vecs = (long long)rows * s.N / 8;
  return (int)((vecs + item_vecs - 1) / item_vecs);
}
MKB_HD int reduce_num_items(const Sched& s, int owner, int item_vecs) {
  return owner_num_items(s, owner) * reduce_chunks_per_piece(s, item_vecs);
}
MKB_HD int choose_item_vecs(const Sched& s, int workers, int min_vecs = 128) {
  // A row-block's rows become reducible all at once (when its last tile lands on the last
  // rank), and the final row-block only at the very end of the GEMM: cut one piece (<= 128 rows)
  // into about one item per worker so that this tail is a single short round for everybody.
  if (workers < 1) workers = 1;
  const int rows = (s.part_rows < kBlockM && !s.one_shot) ? s.part_rows : kBlockM;
  const long long piece = (long long)rows * s.N / 8;
  long long v = (piece + workers - 1) / workers;
  if (v < min_vecs) v = min_vecs;
  if (v > 4096) v = 4096;
  return (int)((v + 31) / 32 * 32);
}

// ------------------------------------------------------------------------------------------
// Work of one compute CTA: whole tiles, then at most one piece of a tail tile.
// ------------------------------------------------------------------------------------------
// Tiles are handed out round-robin (tile t to CTA t mod n_comp), so the last round is usually
// partial: with 6.05 rounds of tiles the 7th keeps 5 % of the CTAs busy for a whole tile time.
// When splitting is enabled (plain GEMM and AllGather+GEMM), the tiles of a partial last round
// are instead cut along K into `parts` pieces, one per CTA (CTA pair), so that every CTA gets a
// share of that round; the pieces' fp32 accumulators go through a scratch buffer and are summed
// in a fixed order (deterministic), each CTA finishing a slice of rows of its tile.
// cg = 1: a unit is a CTA and a tile; cg = 2: a unit is a CTA pair and two consecutive tiles.
struct SplitPlan {
  int full_rounds;   // rounds in which every CTA has a whole tile
  int rem_units;     // tail tiles (pair tiles for cg = 2) = units of the partial round
  int parts;         // pieces per tail tile; 0 = no splitting (the partial round runs whole tiles)
};
MKB_HD SplitPlan plan_split(int total_tiles, int n_comp, int cg, int k_blocks, int max_parts) {
  SplitPlan sp;
  sp.full_rounds = 0; sp.rem_units = 0; sp.parts = 0;
  if (max_parts < 2 || n_comp < cg) return sp;
  const int units = n_comp / cg, unit_tiles = total_tiles / cg;
  const int full = unit_tiles / units, rem = unit_tiles % units;
  if (full < 1 || rem == 0 || rem > units / 2) return sp;
  int parts = units / rem;
  if (parts > max_parts) parts = max_parts;
  if (parts > k_blocks / 4) parts = k_blocks / 4;   // at least four k-blocks per piece
  if (parts < 2) return sp;
  sp.full_rounds = full; sp.rem_units = rem; sp.parts = parts;
  return sp;
}
struct WorkItem {
  int t;          // tile index in visiting order
  int kb0, kb1;   // k-blocks [kb0, kb1)
  int piece;      // -1: the whole tile; else tail tile * parts + part
};
// `cta` = index of this CTA among the compute CTAs, `it` = 0, 1, 2, ... ; false when done.
MKB_HD bool cta_work_item(const SplitPlan& sp, int total_tiles, int n_comp, int cg, int k_blocks,
                          int cta, int it, WorkItem* w) {
  w->kb0 = 0; w->kb1 = k_blocks; w->piece = -1;
  if (sp.parts == 0) {
    w->t = cta + it * n_comp;
    return w->t < total_tiles;
  }
  if (it < sp.full_rounds) { w->t = cta + it * n_comp; return true; }
  if (it > sp.full_rounds) return false;
  const int unit = cta / cg;
  if (unit >= sp.rem_units * sp.parts) return false;
  const int j = unit / sp.parts, i = unit % sp.parts;
  w->t = sp.full_rounds * n_comp + j * cg + (cta % cg);
  w->kb0 = (int)((long long)i * k_blocks / sp.parts);
  w->kb1 = (int)((long long)(i + 1) * k_blocks / sp.parts);
  w->piece = unit;
  return true;
}

// Shared-memory plan for one CTA.
MKB_HD int stage_bytes(int block_n) { return kBlockM * kBlockK * 2 + block_n * kBlockK * 2; }
// Same for a CTA pair (cg = 2): each CTA holds its A tile and half of the B tile.
MKB_HD int stage_bytes_cg(int block_n, int cg) {
  return kBlockM * kBlockK * 2 + (block_n / cg) * kBlockK * 2;
}
// `ring_slots` = 16-byte ring slots per lane of the in-CTA exchange warp (32 -> 16 KB, 96 -> 48 KB).
MKB_HD int smem_fixed_bytes(int ring_slots) {
  return 1024 + kSmemBarrierBytes + kEpilogueStageBytes + ring_slots * 32 * 16;
}
MKB_HD int num_stages_cg(int block_n, int cg, int ring_slots = kRingInCta) {
  int n = (kSmemBudget - smem_fixed_bytes(ring_slots)) / stage_bytes_cg(block_n, cg);
  return n > kMaxStages ? kMaxStages : n;
}
MKB_HD int smem_bytes_cg(int block_n, int cg, int ring_slots = kRingInCta) {
  return smem_fixed_bytes(ring_slots) +
         num_stages_cg(block_n, cg, ring_slots) * stage_bytes_cg(block_n, cg);
}
constexpr int kRingInCtaDeep = 96;     // deeper ring when an operand stage can be given up for it

// Column-block width: pick the multiple of `quantum` in [64, 256] that minimises the number of
// full waves times the tile width (a proxy for time), preferring wider tiles on ties.
// Widths below 128 make the MMA shared-memory bound, so they are considered only when 128-wide
// tiles cannot give every compute CTA a tile (small, latency-bound problems).
MKB_HD int choose_block_n(int M_blocks, int N, int n_compute_ctas, int quantum) {
  int best = 256; long long best_cost = -1;
  const int floor_bn = ((long long)M_blocks * ceil_div(N, 128) < n_compute_ctas) ? 64 : 128;
  for (int bn = 256; bn >= floor_bn; bn -= quantum) {
    const int q = ceil_div(N, bn);
    const long long tiles = (long long)M_blocks * q;
    const long long waves = (tiles + n_compute_ctas - 1) / n_compute_ctas;
    // fixed per-tile overhead (epilogue hand-off, pipeline refill) ~ 24 columns' worth of MMA
    // time; narrower tiles also re-read A more often per output column and run the MMA below
    // its shared-memory-bound rate (measured per-column slowdown: ~1.1x at 192, ~1.35x at 128)
    const long long eff = bn >= 224 ? 100 : bn >= 192 ? 110 : bn >= 128 ? 135 : 160;
    const long long cost = waves * (bn + 24) * eff;
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
  }
  return best;
}

}  // namespace mkb
