// Host side of the operators: argument validation, launch planning, TMA descriptor encoding and
// the extern "C" entry points declared in include/mkernel_b200.h.
//
// Stands in for the reference's host entry points (semantics only):
//   include/operators/ag_gemm/ag_gemm_warp_specialized.cuh:251-406 (globals, config table, launch)
//   src/gemm_rs_blackwell.cu:642-732, include/operators/gemm_ar/gemm_ar_blackwell.cuh:205-246.
// Differences by design: the world size is a run-time value (1..8); unsupported shapes return
// MK_ERR_INVALID instead of silently launching nothing; no call exits the process.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "../../include/mkernel_b200.h"
#include "fused_kernel.cuh"
#include "host_util.h"

namespace mkb {

// ------------------------------------------------------------------------------------------
// options
// ------------------------------------------------------------------------------------------
struct Options {
  long long wait_limit_ms = 4000;
  long long n_comm = -1;   // dedicated exchange CTAs; -1 = heuristic
  long long block_n = 0;
  long long group_rows = 0;
  long long group_cols = 0;   // raster group width in column blocks; 0 = heuristic
  // NVSwitch multicast paths: 0 = never, 1 = whenever the buffers have a multicast alias.
  // Off by default although GEMM+AllReduce at 8 GPUs measured faster with it (42.3 us against
  // 46.0 at the decode shape): the in-switch sum of multimem.ld_reduce is not rounded to nearest
  // (max error 0.0106 of the 1e-2 parity metric at 2 GPUs, against 0.0078 bounded for the fp32
  // sum in the reduce role), and the default path has to hold the parity tolerance.
  long long use_nvls = 0;
  long long debug_flags = 0;  // timing diagnostics; only builds made with -DMKB_DIAG accept it
  long long trace_ptr = 0;    // diagnostics build: device address of 16 counters per CTA
  long long max_stages = 0;   // cap on the operand ring depth (0 = as many as fit)
  long long l2_promo = 3;     // TMA descriptor L2 promotion: 0 none, 1 64 B, 2 128 B, 3 256 B
  // AllGather push pacing, in quarter raster groups (0 = unpaced).  Measured on B200: unpaced
  // pushes arrive long before they are consumed and slow the GEMM on both sides (W=8: 0.504 ms
  // unpaced, 0.445 at 4..8, 0.624 at 2 which starves the consumers; W=2: 0.418 / 0.404 / 0.396).
  long long ag_lead = 6;
  long long ag_fanout = 0;   // AllGather push: load each row group once, store it to every peer
  // AllGather push items: 1 = all rows of a row-block over one K-range (up to 32 ranges per
  // row-block, pushed range-major), and the consumer's TMA producer waits range by range inside
  // its K loop, so a tile starts when 1/32 of its rows' bytes have landed; 0 = 4 full rows per
  // item and the consumer waits for the whole row-block.  The single-destination store path
  // only: the fan-out, multicast and bulk-store variants keep the row form.
  long long ag_chunks = 0;
  long long push_bulk = 0;   // AllGather push through TMA bulk stores instead of LSU stores
  long long ar_one_shot = 0;  // GEMM+AR: 1 = every rank reduces all rows itself (no broadcast)
  // GEMM+AR two-shot: the epilogue also stores partial rows into their owner's staging slabs
  // (posted remote stores) and owners reduce from local memory, when the output fits the slabs.
  // 2 = every 32-bit data word is stored together with the epoch, so owners need no flags and no
  // fences (M x N <= 1 Mi elements, else as 1); 1 = plain slabs plus per-tile flags (M x N <=
  // 2 Mi elements, else as 0); 0 = owners always fetch the partials from their producers.
  long long ar_push = 2;
  long long cta_pair = 1;   // 1: run compute CTAs as pairs (two-SM MMA) when the shape allows
  // 1: launch with programmatic stream serialization, so that a kernel's set-up (barriers, tensor
  // memory) overlaps the tail of the previous kernel in the stream; the reference launches the
  // same way (src/gemm_rs_blackwell.cu:668-680, src/ag_gemm_warp_specialized.cu:678-690).
  long long pdl = 1;
  // 1: cut the tiles of a partial last round along K over all CTAs (plain GEMM and
  // AllGather+GEMM); needs a per-stream scratch buffer the library allocates on first use.
  long long split_tail = 1;
};
static Options g_opt;
static std::mutex g_opt_mu;

static long long* option_slot(const char* name) {
  if (!name) return nullptr;
  if (!strcmp(name, "wait_limit_ms")) return &g_opt.wait_limit_ms;
  if (!strcmp(name, "n_comm")) return &g_opt.n_comm;
  if (!strcmp(name, "block_n")) return &g_opt.block_n;
  if (!strcmp(name, "group_rows")) return &g_opt.group_rows;
  if (!strcmp(name, "group_cols")) return &g_opt.group_cols;
  if (!strcmp(name, "use_nvls")) return &g_opt.use_nvls;
  if (!strcmp(name, "cta_pair")) return &g_opt.cta_pair;
  if (!strcmp(name, "pdl")) return &g_opt.pdl;
  if (!strcmp(name, "split_tail")) return &g_opt.split_tail;
#ifdef MKB_DIAG
  if (!strcmp(name, "debug_flags")) return &g_opt.debug_flags;
  if (!strcmp(name, "trace_ptr")) return &g_opt.trace_ptr;
#endif
  if (!strcmp(name, "max_stages")) return &g_opt.max_stages;
  if (!strcmp(name, "l2_promo")) return &g_opt.l2_promo;
  if (!strcmp(name, "push_bulk")) return &g_opt.push_bulk;
  if (!strcmp(name, "ag_fanout")) return &g_opt.ag_fanout;
  if (!strcmp(name, "ag_lead")) return &g_opt.ag_lead;
  if (!strcmp(name, "ag_chunks")) return &g_opt.ag_chunks;
  if (!strcmp(name, "ar_one_shot")) return &g_opt.ar_one_shot;
  if (!strcmp(name, "ar_push")) return &g_opt.ar_push;
  return nullptr;
}

// Range check shared by mk_set_option and the environment parser.  Only n_comm accepts -1
// (= heuristic); the device wait budget stays within [1 ms, 60 s] so that no configuration can
// turn the bounded waits into unbounded ones.
static const char* option_range_error(const char* name, long long v) {
  if (!strcmp(name, "n_comm")) return v >= -1 && v <= 147 ? nullptr : "must be in [-1, 147]";
  if (!strcmp(name, "wait_limit_ms")) return v >= 1 && v <= 60000 ? nullptr : "must be in [1, 60000]";
  if (!strcmp(name, "block_n")) return v >= 0 && v <= 256 ? nullptr : "must be in [0, 256]";
  if (!strcmp(name, "max_stages")) return v >= 0 && v <= kMaxStages ? nullptr : "must be in [0, 8]";
  if (!strcmp(name, "l2_promo")) return v >= 0 && v <= 3 ? nullptr : "must be in [0, 3]";
  if (!strcmp(name, "group_rows") || !strcmp(name, "group_cols") || !strcmp(name, "ag_lead"))
    return v >= 0 && v <= 4096 ? nullptr : "must be in [0, 4096]";
  if (!strcmp(name, "trace_ptr")) return nullptr;
  if (!strcmp(name, "debug_flags")) return v >= 0 && v <= 0xffff ? nullptr : "must be in [0, 65535]";
  if (!strcmp(name, "ar_push")) return v >= 0 && v <= 2 ? nullptr : "must be 0, 1 or 2";
  return v >= 0 && v <= 1 ? nullptr : "must be 0 or 1";
}

// Start-up defaults from the environment, for callers that cannot reach mk_set_option (a launcher
// script around an unmodified host program): MKERNEL_B200_OPTIONS="use_nvls=1,block_n=256".
// Unknown names and malformed entries are reported on stderr and skipped.
struct EnvOptions {
  EnvOptions() {
    const char* env = getenv("MKERNEL_B200_OPTIONS");
    if (!env || !*env) return;
    std::string all(env);
    size_t pos = 0;
    while (pos <= all.size()) {
      size_t end = all.find(',', pos);
      if (end == std::string::npos) end = all.size();
      const std::string item = all.substr(pos, end - pos);
      pos = end + 1;
      if (item.empty()) continue;
      const size_t eq = item.find('=');
      const std::string name = eq == std::string::npos ? std::string() : item.substr(0, eq);
      long long* slot = eq == std::string::npos ? nullptr : option_slot(name.c_str());
      char* tail = nullptr;
      const long long v = eq == std::string::npos ? 0 : strtoll(item.c_str() + eq + 1, &tail, 10);
      if (!slot || !tail || *tail != 0 || tail == item.c_str() + eq + 1 ||
          option_range_error(name.c_str(), v) != nullptr) {
        fprintf(stderr, "mkernel_b200: ignoring MKERNEL_B200_OPTIONS entry '%s'\n", item.c_str());
        continue;
      }
      *slot = v;
    }
  }
};
static EnvOptions g_env_options;

// ------------------------------------------------------------------------------------------
// planning (pure host arithmetic; also exported for tests)
// ------------------------------------------------------------------------------------------
struct Plan {
  Sched sched;
  int K, k_blocks, stages, n_comm, grid, smem;
  int cg;   // 1: independent CTAs; 2: CTA pairs
  int ring_slots;
  int b_mn_major;
};

static int default_n_comm(int op, int world, int M, int N, int K, int num_sms) {
  // Every compute CTA carries one exchange warp.  Dedicated exchange CTAs (8 workers each) can be
  // requested with the n_comm option; measured on B200 they did not help, not even for the
  // decode-shaped AllReduce (more workers contend on the item queue and on system-scope fences:
  // 21 us against 15 us for the reduce phase at W = 4), so the default is none.
  (void)op; (void)world; (void)M; (void)N; (void)K; (void)num_sms;
  return 0;
}

static Options options_snapshot() {
  std::lock_guard<std::mutex> g(g_opt_mu);
  return g_opt;
}

static int make_plan(const Options& o, int op, int rank, int world, int M, int N, int K,
                     int b_layout, int num_sms, Plan* out, int epilogue = EPI_NONE) {
  if (op < OP_GEMM || op > OP_AR) return set_error(MK_ERR_INVALID, "unknown op %d", op);
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world)
    return set_error(MK_ERR_INVALID, "rank/world out of range: rank=%d world=%d", rank, world);
  if (M < 1 || N < 1 || K < 1)
    return set_error(MK_ERR_INVALID, "M, N, K must be positive (M=%d N=%d K=%d)", M, N, K);
  if (N % 8 != 0 || K % 8 != 0)
    return set_error(MK_ERR_INVALID, "N and K must be multiples of 8 (N=%d K=%d)", N, K);
  if (op == OP_AG && M % world != 0)
    return set_error(MK_ERR_INVALID, "AllGather+GEMM: M=%d not divisible by world=%d", M, world);
  if (op == OP_RS && M % world != 0)
    return set_error(MK_ERR_INVALID, "GEMM+ReduceScatter: M=%d not divisible by world=%d", M, world);
  if (num_sms <= 0) num_sms = 148;

  int n_comm = (int)o.n_comm >= 0 && world > 1 && op != OP_GEMM
                   ? (int)o.n_comm : default_n_comm(op, world, M, N, K, num_sms);
  if (n_comm > num_sms - 1) n_comm = num_sms - 1;
  const int n_comp_max = num_sms - n_comm;

  int m_blocks = op == OP_AG ? world * ceil_div(M / world, kBlockM) : ceil_div(M, kBlockM);
  // CTA pairs (two-SM MMA) need an even number of row-blocks and pay off only when the GEMM
  // fills the machine; halves that are not multiples of 64 columns run the tensor pipe poorly,
  // so pair mode picks the tile width among multiples of 128.
  const bool pair_ok = o.cta_pair != 0 && m_blocks % 2 == 0 && n_comm % 2 == 0 && n_comp_max >= 2 &&
                       (long long)m_blocks * ceil_div(N, 128) >= n_comp_max;
  const int quantum = pair_ok ? 128 : (b_layout == MK_B_KN ? 64 : 32);
  int bn = (int)o.block_n;
  if (epilogue == EPI_SWIGLU) {
    // a tile is 128 gate columns followed by the 128 up columns of the same outputs
    if (op != OP_GEMM && op != OP_AG)
      return set_error(MK_ERR_INVALID, "the SwiGLU epilogue exists for GEMM and AllGather+GEMM only");
    if (N % 256 != 0 || b_layout != MK_B_NK)
      return set_error(MK_ERR_INVALID, "SwiGLU epilogue: N=%d must be a multiple of 256 and B "
                       "stored [N, K] with 128 gate rows then 128 up rows per 256-row block", N);
    bn = 256;
  }
  if (bn <= 0) bn = choose_block_n(m_blocks, N, n_comp_max, quantum);
  const int min_q = b_layout == MK_B_KN ? 64 : 32;
  if (bn < 32 || bn > 256 || bn % min_q != 0)
    return set_error(MK_ERR_INVALID, "block_n=%d must be a multiple of %d in [32,256]", bn, min_q);

  // Raster group height: tiles are visited in groups of `group` row-blocks, row-block fastest,
  // so a group's A rows (group x 128 x K) stay in L2 while B streams past once per group.
  // One GPU: ~16-30 MB of A per group measured best (8 row-blocks at K=8192, up to 32 at
  // K=3584).  With an exchange running, 8 (one shard / one owner round at W=8) measured best.
  int group = (int)o.group_rows;
  if (group <= 0) {
    group = 8;
    if (world > 1 && op == OP_AG) {
      // AllGather+GEMM: 12 row-blocks where a shard has at least that many (measured at two
      // GPUs with 32 blocks per shard: 4-6 % faster than 8); never more than one shard, which
      // at eight GPUs and 8192 rows is 8 blocks.
      if (ceil_div(M / world, kBlockM) >= 12) group = 12;
    }
    if (world == 1) {
      const long long rb_bytes = (long long)kBlockM * K * 2;
      long long g = (24LL << 20) / (rb_bytes > 0 ? rb_bytes : 1);
      g &= ~1LL;
      if (g < 8) g = 8;
      if (g > 32) g = 32;
      group = (int)g;
    }
  }
  Plan pl;
  pl.sched = make_sched(op, rank, world, M, N, bn, group, (int)o.group_cols);
  if (op == OP_AR && world > 1 && o.ar_one_shot != 0) {
    pl.sched.one_shot = 1;
    pl.sched.interleave = 0;
  }
  pl.K = K;
  pl.k_blocks = ceil_div(K, kBlockK);
  pl.b_mn_major = b_layout == MK_B_KN ? 1 : 0;
  const long long tiles = (long long)pl.sched.P * pl.sched.Q;
  int n_comp = tiles < n_comp_max ? (int)tiles : n_comp_max;
  if (n_comp < 1) n_comp = 1;
  // CTA pairs: consecutive tiles (2i, 2i+1) must share a column block, which holds when every
  // raster group has an even number of row-blocks; the pair splits B's rows in two halves.
  pl.cg = 1;
  if (pair_ok && pl.sched.P % 2 == 0 && pl.sched.group_rows % 2 == 0 && tiles >= 2 &&
      bn % (pl.b_mn_major ? 128 : 32) == 0 && (n_comp & ~1) >= 2) {
    pl.cg = 2;
    n_comp &= ~1;
  }
  // With an exchange to feed, trade one operand stage for a three times deeper ring of the
  // in-CTA exchange warp (its throughput is bytes in flight / memory latency) when at least
  // five stages remain.
  pl.ring_slots = kRingInCta;
  if (world > 1 && op != OP_GEMM && num_stages_cg(bn, pl.cg, kRingInCtaDeep) >= 5)
    pl.ring_slots = kRingInCtaDeep;
  pl.stages = num_stages_cg(bn, pl.cg, pl.ring_slots);
  pl.smem = smem_bytes_cg(bn, pl.cg, pl.ring_slots);
  if (o.max_stages >= 2 && pl.stages > (int)o.max_stages) pl.stages = (int)o.max_stages;
  // a dedicated exchange CTA lays 8 warp rings over the stage region and what follows it
  if (pl.smem < 1024 + kSmemBarrierBytes + 8 * kRingDedicated * 32 * 16)
    return set_error(MK_ERR_INVALID, "internal: shared-memory plan too small for exchange rings");
  pl.n_comm = n_comm;
  pl.grid = n_comm + n_comp;
  *out = pl;
  return MK_OK;
}

// ------------------------------------------------------------------------------------------
// TMA descriptors
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Encoding a descriptor costs a few microseconds of host time, which matters for the
// latency-bound shapes; the last few descriptors are kept per thread, keyed by all inputs.
struct MapKey {
  const void* base;
  uint64_t inner, outer, ld;
  uint32_t box_inner, box_outer;
  int promo;
  bool operator==(const MapKey& o) const {
    return base == o.base && inner == o.inner && outer == o.outer && ld == o.ld &&
           box_inner == o.box_inner && box_outer == o.box_outer && promo == o.promo;
  }
};
struct MapCache {
  static constexpr int kSlots = 16;
  MapKey key[kSlots];
  CUtensorMap map[kSlots];
  bool used[kSlots] = {};
  int next = 0;
};

static int encode_2d_bf16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer,
                          uint64_t ld_elems, uint32_t box_inner, uint32_t box_outer, int promo) {
  static thread_local MapCache cache;
  const MapKey k{base, inner, outer, ld_elems, box_inner, box_outer, promo};
  for (int i = 0; i < MapCache::kSlots; ++i) {
    if (cache.used[i] && cache.key[i] == k) { *map = cache.map[i]; return MK_OK; }
  }
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    int rc = driver_entry("cuTensorMapEncodeTiled", &p);
    if (rc != MK_OK) return rc;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld_elems * 2) % 16 != 0)
    return set_error(MK_ERR_INVALID, "operand base/stride must be 16-byte aligned");
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {ld_elems * 2};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  static_cast<CUtensorMapL2promotion>(promo), CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(MK_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  cache.key[cache.next] = k;
  cache.map[cache.next] = *map;
  cache.used[cache.next] = true;
  cache.next = (cache.next + 1) % MapCache::kSlots;
  return MK_OK;
}

// ------------------------------------------------------------------------------------------
// launch
// ------------------------------------------------------------------------------------------
static int device_sm_count(int* out) {
  static int cached[64];
  int dev = 0;
  MKB_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && cached[dev] > 0) { *out = cached[dev]; return MK_OK; }
  int n = 0;
  MKB_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
  int major = 0;
  MKB_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10)
    return set_error(MK_ERR_UNSUPPORTED, "device compute capability %d.x is not sm_100", major);
  if (dev >= 0 && dev < 64) cached[dev] = n;
  *out = n;
  return MK_OK;
}

template <int OP, int CG>
static int launch_kernel(const Plan& pl, const CUtensorMap& ta, const CUtensorMap& tb,
                         const OpParams& p, cudaStream_t stream, bool pdl) {
  auto kern = fused_gemm_kernel<OP, CG>;
  static bool attr_set[64];
  int dev = 0;
  MKB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    MKB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pl.grid, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (CG == 2) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 2;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  if (pdl) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = n_attr ? attr : nullptr;
  cfg.numAttrs = n_attr;
  if (CG == 2) {
    // The kernel is persistent and its roles wait on one another, so every CTA must be resident
    // at once: never launch more pairs than the device can hold (SM counts per GPC need not be
    // even, which can leave an SM without a partner).
    static int max_pairs[64];
    if (dev < 0 || dev >= 64 || max_pairs[dev] == 0) {
      int n = 0;
      cudaLaunchConfig_t occ = cfg;       // the occupancy query takes the cluster attribute only
      occ.numAttrs = 1;
      MKB_CUDA(cudaOccupancyMaxActiveClusters(&n, kern, &occ));
      if (n < 1) return set_error(MK_ERR_CUDA, "device cannot co-schedule a CTA pair");
      if (dev >= 0 && dev < 64) max_pairs[dev] = n;
      if (pl.grid / 2 > n) cfg.gridDim = dim3(2 * n, 1, 1);
    } else if (pl.grid / 2 > max_pairs[dev]) {
      cfg.gridDim = dim3(2 * max_pairs[dev], 1, 1);
    }
    if ((int)cfg.gridDim.x <= p.n_comm)
      return set_error(MK_ERR_INVALID, "no SM pair left for the GEMM role");
  }
  MKB_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, tb, p));
  return MK_OK;
}

// ------------------------------------------------------------------------------------------
// scratch for split tail tiles
// ------------------------------------------------------------------------------------------
// One buffer per (device, stream), allocated on first use and kept: launches on one stream are
// serialised, so they can share it; launches on different streams may overlap and must not.
// Layout: 4 KiB of arrival counters, then one 128 x 256 fp32 slot per SM.  The reference keeps
// hidden per-device scratch the same way (include/operators/gemm_rs/gemm_rs.cuh:428-475).
// Returns nullptr (splitting stays off for this launch) when the stream is being captured and
// has no buffer yet, when the cache is full, or when the allocation fails.
constexpr size_t kSplitCounterBytes = 4096;
static char* split_scratch_for(cudaStream_t stream, int num_sms) {
  struct Entry { int dev; cudaStream_t stream; char* ptr; };
  static Entry cache[16];
  static int n_cached = 0;
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> g(mu);
  for (int i = 0; i < n_cached; ++i)
    if (cache[i].dev == dev && cache[i].stream == stream) return cache[i].ptr;
  if (n_cached == 16) return nullptr;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return nullptr;
  }
  void* ptr = nullptr;
  const size_t bytes = kSplitCounterBytes + (size_t)num_sms * kBlockM * 256 * 4;
  if (cudaMalloc(&ptr, bytes) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  if (cudaMemset(ptr, 0, kSplitCounterBytes) != cudaSuccess) { cudaGetLastError(); cudaFree(ptr); return nullptr; }
  cache[n_cached++] = Entry{dev, stream, static_cast<char*>(ptr)};
  return static_cast<char*>(ptr);
}

struct OpArgs {
  int op;
  const void* A;       // GEMM A operand (AG: local gathered buffer)
  long long a_rows;    // rows addressable through the A descriptor
  const void* B;
  void* C;
  int M, N, K, b_layout;
  int rank, world;
  const mk_symm_view* sync;
  const mk_symm_view* data;   // AG: A; RS/AR: C
  const mk_symm_view* out;    // AR: C_final
  uint32_t epoch;
  uint32_t* status_only;      // plain GEMM: optional 4 status words
  int epilogue;               // Epilogue (EPI_NONE unless stated)
};

static int run_op(const OpArgs& a, cudaStream_t stream) {
  int sms = 0;
  int rc = device_sm_count(&sms);
  if (rc != MK_OK) return rc;
  const Options o = options_snapshot();
  Plan pl;
  rc = make_plan(o, a.op, a.rank, a.world, a.M, a.N, a.K, a.b_layout, sms, &pl, a.epilogue);
  if (rc != MK_OK) return rc;

  OpParams p;
  memset(&p, 0, sizeof(p));
  p.sched = pl.sched;
  p.K = a.K;
  p.k_blocks = pl.k_blocks;
  p.stages = pl.stages;
  p.b_mn_major = pl.b_mn_major;
  p.n_comm = pl.n_comm;
  p.ring_slots = pl.ring_slots;
  const bool want_nvls = o.use_nvls != 0;
  p.debug_flags = (int)o.debug_flags;
  p.trace = reinterpret_cast<unsigned long long*>(static_cast<uintptr_t>(o.trace_ptr));
  p.push_bulk = (int)o.push_bulk;
  p.ag_fanout = (int)o.ag_fanout;
  p.ag_lead_tiles = (int)(o.ag_lead * pl.sched.group_rows * pl.sched.Q / 4);
  if (a.op == OP_AG && a.world > 1 && o.ag_chunks != 0 && !p.push_bulk && !p.ag_fanout &&
      !(want_nvls && a.data && a.data->mc != nullptr)) {
    // K-range of an item: the smallest power of two of 16-byte vectors, at least one k-block
    // (8 vectors), that covers a row in at most kGatherSub ranges.
    const int row_vecs = a.K / 8;
    int lg = 3;
    while ((kGatherSub << lg) < row_vecs) ++lg;
    p.ag_cv_log2 = lg;
  }
  if (a.sync && a.op == OP_AR && o.ar_push != 0 && !want_nvls &&
      sync_words_needed(pl.sched) * 4 <= kArSlabByteOffset) {
    if (o.ar_push >= 2 && ar_push_fits(pl.sched, (long long)a.sync->bytes, 2)) pl.sched.ar_push = 2;
    else if (ar_push_fits(pl.sched, (long long)a.sync->bytes, 1)) pl.sched.ar_push = 1;
  }
  p.sched = pl.sched;
  if (a.world > 1 && a.op != OP_GEMM) {
    // Exchange workers: one warp per compute CTA (eight per dedicated exchange CTA).  With the
    // epoch-carrying slabs of the latency-bound AllReduce every warp of a CTA turns into a worker
    // once its GEMM role has finished, and a piece is cut accordingly finer.
    const bool all_warps = a.op == OP_AR && pl.sched.ar_push == 2;
    const int workers = (all_warps ? 8 : 1) * (pl.grid - pl.n_comm) + 8 * pl.n_comm;
    if (a.op == OP_AG) {
      p.item_vecs = 0;
      p.n_items = gather_num_items(pl.sched, p.ag_fanout != 0 ||
                                                 (want_nvls && a.data && a.data->mc != nullptr));
    } else {
      p.item_vecs = choose_item_vecs(pl.sched, workers, all_warps ? 32 : 128);
      p.n_items = reduce_num_items(pl.sched, a.rank, p.item_vecs);
    }
  }
  p.epoch_arg = a.epoch;
  p.wait_limit_ns = (uint64_t)o.wait_limit_ms * 1000000ull;
  p.use_nvls = want_nvls ? 1 : 0;
  p.C = a.C;
  p.epilogue = a.epilogue;
  p.ldc = a.epilogue == EPI_SWIGLU ? a.N / 2 : a.N;
  if (a.sync) {
    const long long need = sync_words_needed(pl.sched);
    if ((long long)(a.sync->bytes / 4) < need)
      return set_error(MK_ERR_INVALID, "synchronisation buffer holds %lld words, this shape needs %lld",
                       (long long)(a.sync->bytes / 4), need);
    p.sync = static_cast<uint32_t*>(a.sync->peer[a.rank]);
    p.status = p.sync + SW_STATUS;
    for (int r = 0; r < a.world; ++r) p.peer_sync[r] = static_cast<uint32_t*>(a.sync->peer[r]);
  } else {
    // The plain GEMM has no synchronisation buffer; it can still report a pipeline timeout
    // through 4 caller-provided words laid out like SW_STATUS.
    p.sync = nullptr;
    p.status = a.status_only;
  }
  if (a.data) {
    for (int r = 0; r < a.world; ++r) p.peer_data[r] = a.data->peer[r];
    p.mc_data = a.data->mc;
  }
  if (a.out) {
    for (int r = 0; r < a.world; ++r) p.peer_out[r] = a.out->peer[r];
    p.mc_out = a.out->mc;
  }
  for (int r = 0; r < a.world; ++r) {
    if ((a.sync && !p.peer_sync[r]) || (a.data && !p.peer_data[r]) || (a.out && !p.peer_out[r]))
      return set_error(MK_ERR_INVALID, "symmetric view has no address for rank %d", r);
  }

  // Split tail tiles (plain GEMM, AllGather+GEMM): the kernel decides from its actual grid
  // whether the last round is partial enough; here it only gets the scratch and clean counters.
  if ((a.op == OP_GEMM || a.op == OP_AG) && o.split_tail != 0 && pl.n_comm == 0 &&
      (long long)pl.sched.P * pl.sched.Q > pl.grid && pl.k_blocks >= 8) {
    const int units = pl.grid / pl.cg;
    const long long unit_tiles = (long long)pl.sched.P * pl.sched.Q / pl.cg;
    const int rem = (int)(unit_tiles % units);
    if (rem != 0 && rem <= units / 2) {
      if (char* scratch = split_scratch_for(stream, sms)) {
        MKB_CUDA(cudaMemsetAsync(scratch, 0, kSplitCounterBytes, stream));
        p.split_counters = reinterpret_cast<uint32_t*>(scratch);
        p.split_scratch = reinterpret_cast<float*>(scratch + kSplitCounterBytes);
        p.split_max_parts = 32;
      }
    }
  }

  CUtensorMap ta, tb;
  const int promo = (int)o.l2_promo;
  rc = encode_2d_bf16(&ta, a.A, (uint64_t)a.K, (uint64_t)a.a_rows, (uint64_t)a.K, kBlockK, kBlockM,
                      promo);
  if (rc != MK_OK) return rc;
  if (pl.b_mn_major)
    rc = encode_2d_bf16(&tb, a.B, (uint64_t)a.N, (uint64_t)a.K, (uint64_t)a.N, 64, kBlockK, promo);
  else
    rc = encode_2d_bf16(&tb, a.B, (uint64_t)a.K, (uint64_t)a.N, (uint64_t)a.K, kBlockK,
                        (uint32_t)(pl.sched.block_n / pl.cg), promo);
  if (rc != MK_OK) return rc;
  if ((reinterpret_cast<uintptr_t>(a.C) & 15) != 0)
    return set_error(MK_ERR_INVALID, "C must be 16-byte aligned");

  if (pl.cg == 2) {
    switch (a.op) {
      case OP_GEMM: return launch_kernel<OP_GEMM, 2>(pl, ta, tb, p, stream, o.pdl != 0);
      case OP_AG: return launch_kernel<OP_AG, 2>(pl, ta, tb, p, stream, o.pdl != 0);
      case OP_RS: return launch_kernel<OP_RS, 2>(pl, ta, tb, p, stream, o.pdl != 0);
      case OP_AR: return launch_kernel<OP_AR, 2>(pl, ta, tb, p, stream, o.pdl != 0);
    }
  }
  switch (a.op) {
    case OP_GEMM: return launch_kernel<OP_GEMM, 1>(pl, ta, tb, p, stream, o.pdl != 0);
    case OP_AG: return launch_kernel<OP_AG, 1>(pl, ta, tb, p, stream, o.pdl != 0);
    case OP_RS: return launch_kernel<OP_RS, 1>(pl, ta, tb, p, stream, o.pdl != 0);
    case OP_AR: return launch_kernel<OP_AR, 1>(pl, ta, tb, p, stream, o.pdl != 0);
  }
  return set_error(MK_ERR_INVALID, "unknown op");
}

static int check_view(const mk_symm_view* v, const char* what, size_t min_bytes) {
  if (!v) return set_error(MK_ERR_INVALID, "%s: null symmetric view", what);
  if (v->world < 1 || v->world > kMaxWorld || v->rank < 0 || v->rank >= v->world)
    return set_error(MK_ERR_INVALID, "%s: bad rank/world %d/%d", what, v->rank, v->world);
  if (v->bytes < min_bytes)
    return set_error(MK_ERR_INVALID, "%s: %zu bytes, need at least %zu", what, v->bytes, min_bytes);
  if (!v->peer[v->rank]) return set_error(MK_ERR_INVALID, "%s: no local address", what);
  return MK_OK;
}

}  // namespace mkb

using namespace mkb;

// ------------------------------------------------------------------------------------------
// extern "C"
// ------------------------------------------------------------------------------------------
extern "C" {

int mk_version(void) { return 100; }

int mk_set_option(const char* name, long long value) {
  std::lock_guard<std::mutex> g(g_opt_mu);
  long long* s = option_slot(name);
  if (!s) return set_error(MK_ERR_INVALID, "unknown option '%s'", name ? name : "(null)");
  if (const char* why = option_range_error(name, value))
    return set_error(MK_ERR_INVALID, "option '%s' %s (got %lld)", name, why, value);
  *s = value;
  return MK_OK;
}

long long mk_get_option(const char* name) {
  std::lock_guard<std::mutex> g(g_opt_mu);
  long long* s = option_slot(name);
  return s ? *s : -1;
}

int mk_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int b_layout,
                 uint32_t* status4, void* stream) {
  if (!A || !B || !C) return set_error(MK_ERR_INVALID, "mk_gemm_bf16: null operand");
  OpArgs a;
  memset(&a, 0, sizeof(a));
  a.op = OP_GEMM; a.A = A; a.a_rows = M; a.B = B; a.C = C;
  a.M = M; a.N = N; a.K = K; a.b_layout = b_layout; a.rank = 0; a.world = 1;
  a.status_only = status4;
  return run_op(a, static_cast<cudaStream_t>(stream));
}

int mk_ag_gemm_prepare(const mk_symm_view* ready, void* stream) {
  // The reference runs an all-rank barrier kernel here (src/ag_gemm_warp_specialized.cu:115-134).
  // In this design the launch itself carries the ordering: every rank announces "entered launch
  // e" to its peers when its kernel starts, and nobody writes into a peer's gathered buffer
  // before seeing that announcement.  prepare therefore only validates its argument; it is kept
  // so that callers written against the reference run unchanged.
  (void)stream;
  return check_view(ready, "ready", (size_t)MK_AG_READY_WORDS * 4);
}

int mk_ag_gemm_launch(const mk_symm_view* A, const mk_symm_view* ready, const void* B, void* C,
                      int M, int N, int K, void* stream) {
  return mk_ag_gemm_launch_ex(A, ready, B, C, M, N, K, MK_B_NK, 0, stream);
}

int mk_ag_gemm_launch_ex(const mk_symm_view* A, const mk_symm_view* ready, const void* B, void* C,
                         int M, int N, int K, int b_layout, uint32_t epoch, void* stream) {
  if (!B || !C) return set_error(MK_ERR_INVALID, "mk_ag_gemm_launch: null operand");
  if (b_layout != MK_B_KN && b_layout != MK_B_NK)
    return set_error(MK_ERR_INVALID, "mk_ag_gemm_launch: unknown B layout %d", b_layout);
  if (M < 1 || K < 1) return set_error(MK_ERR_INVALID, "mk_ag_gemm_launch: bad shape");
  int rc = check_view(A, "A", (size_t)M * K * 2);
  if (rc != MK_OK) return rc;
  rc = check_view(ready, "ready", (size_t)MK_AG_READY_WORDS * 4);
  if (rc != MK_OK) return rc;
  if (A->world != ready->world || A->rank != ready->rank)
    return set_error(MK_ERR_INVALID, "A and ready disagree on rank/world");
  OpArgs a;
  memset(&a, 0, sizeof(a));
  a.op = OP_AG; a.A = A->peer[A->rank]; a.a_rows = M; a.B = B; a.C = C;
  a.M = M; a.N = N; a.K = K; a.b_layout = b_layout; a.rank = A->rank; a.world = A->world;
  a.sync = ready; a.data = A; a.epoch = epoch;
  return run_op(a, static_cast<cudaStream_t>(stream));
}

int mk_ag_gemm_swiglu_launch(const mk_symm_view* A, const mk_symm_view* ready,
                             const void* B_gate_up, void* H, int M, int N2, int K, void* stream) {
  if (!B_gate_up || !H) return set_error(MK_ERR_INVALID, "mk_ag_gemm_swiglu_launch: null operand");
  if (M < 1 || K < 1 || N2 < 256)
    return set_error(MK_ERR_INVALID, "mk_ag_gemm_swiglu_launch: bad shape");
  int rc = check_view(A, "A", (size_t)M * K * 2);
  if (rc != MK_OK) return rc;
  rc = check_view(ready, "ready", (size_t)MK_AG_READY_WORDS * 4);
  if (rc != MK_OK) return rc;
  if (A->world != ready->world || A->rank != ready->rank)
    return set_error(MK_ERR_INVALID, "A and ready disagree on rank/world");
  OpArgs a;
  memset(&a, 0, sizeof(a));
  a.op = OP_AG; a.A = A->peer[A->rank]; a.a_rows = M; a.B = B_gate_up; a.C = H;
  a.M = M; a.N = N2; a.K = K; a.b_layout = MK_B_NK; a.rank = A->rank; a.world = A->world;
  a.sync = ready; a.data = A; a.epilogue = EPI_SWIGLU;
  return run_op(a, static_cast<cudaStream_t>(stream));
}

int mk_gemm_rs_prepare(const mk_symm_view* sync, void* stream) {
  int rc = check_view(sync, "sync", (size_t)MK_RS_SYNC_WORDS * 4);
  if (rc != MK_OK) return rc;
  MKB_CUDA(cudaMemsetAsync(sync->peer[sync->rank], 0, sync->bytes, static_cast<cudaStream_t>(stream)));
  return MK_OK;
}

int mk_gemm_rs_launch(const void* A, const void* B, const mk_symm_view* C,
                      const mk_symm_view* sync, int M, int N, int K, void* stream) {
  return mk_gemm_rs_launch_ex(A, B, C, sync, M, N, K, MK_B_NK, 0, stream);
}

int mk_gemm_rs_launch_ex(const void* A, const void* B, const mk_symm_view* C,
                         const mk_symm_view* sync, int M, int N, int K, int b_layout,
                         uint32_t epoch, void* stream) {
  if (!A || !B) return set_error(MK_ERR_INVALID, "mk_gemm_rs_launch: null operand");
  if (b_layout != MK_B_KN && b_layout != MK_B_NK)
    return set_error(MK_ERR_INVALID, "mk_gemm_rs_launch: unknown B layout %d", b_layout);
  if (M < 1 || N < 1) return set_error(MK_ERR_INVALID, "mk_gemm_rs_launch: bad shape");
  int rc = check_view(C, "C", (size_t)M * N * 2);
  if (rc != MK_OK) return rc;
  rc = check_view(sync, "sync", (size_t)SW_FLAGS * 4);
  if (rc != MK_OK) return rc;
  if (C->world != sync->world || C->rank != sync->rank)
    return set_error(MK_ERR_INVALID, "C and sync disagree on rank/world");
  OpArgs a;
  memset(&a, 0, sizeof(a));
  a.op = OP_RS; a.A = A; a.a_rows = M; a.B = B; a.C = C->peer[C->rank];
  a.M = M; a.N = N; a.K = K; a.b_layout = b_layout; a.rank = C->rank; a.world = C->world;
  a.sync = sync; a.data = C; a.epoch = epoch;
  return run_op(a, static_cast<cudaStream_t>(stream));
}

// ---- one-GPU GEMM+ReduceScatter that allocates nothing --------------------------------------
// The synchronisation words the kernel needs (epoch, CTA counters, status) normally live in a
// buffer the caller allocates.  Some callers cannot allocate device memory at the point where
// they need the product: code running inside a pre-planned memory arena that owns every byte of
// the GPU (an inference server that sized its pools at start-up), or code on a path where
// cudaMalloc's implicit device synchronisation is not acceptable.  For them the words live in
// this file-scope device array, which every GPU that loads the library holds until exit.
// In host code the array's name is only a handle for the runtime, not a device address: the
// address is looked up once per device with cudaGetSymbolAddress and that pointer is what the
// kernel receives.
constexpr int kNoAllocSyncWords = 16384;  // 64 KiB: header (64 words) + one word per output
                                          // tile + one per row-block
static __device__ __align__(256) uint32_t g_noalloc_sync_words[kNoAllocSyncWords];

static int noalloc_sync_address(uint32_t** out) {
  static uint32_t* per_device[64];
  static std::mutex mu;
  int dev = 0;
  MKB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(MK_ERR_INVALID, "device index %d out of range", dev);
  std::lock_guard<std::mutex> g(mu);
  if (per_device[dev] == nullptr) {
    void* p = nullptr;
    MKB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_sync_words));
    if (p == nullptr) return set_error(MK_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    per_device[dev] = static_cast<uint32_t*>(p);
  }
  *out = per_device[dev];
  return MK_OK;
}

int mk_gemm_rs_launch_noalloc(const void* A, const void* B, void* C, int M, int N, int K,
                              void* stream) {
  if (!A || !B || !C) return set_error(MK_ERR_INVALID, "mk_gemm_rs_launch_noalloc: null operand");
  int sms = 0;
  int rc = device_sm_count(&sms);
  if (rc != MK_OK) return rc;
  Plan pl;
  rc = make_plan(options_snapshot(), OP_RS, 0, 1, M, N, K, MK_B_NK, sms, &pl);
  if (rc != MK_OK) return rc;
  const long long need = sync_words_needed(pl.sched);
  if (need > kNoAllocSyncWords)
    return set_error(MK_ERR_INVALID,
                     "mk_gemm_rs_launch_noalloc: %d x %d output needs %lld synchronisation words, "
                     "the built-in buffer holds %d (tiles plus row-blocks at most %d); use "
                     "mk_gemm_rs_launch with a caller-provided buffer",
                     M, N, need, kNoAllocSyncWords, kNoAllocSyncWords - SW_FLAGS);
  uint32_t* words = nullptr;
  rc = noalloc_sync_address(&words);  // first call on a device: looks the address up
  if (rc != MK_OK) return rc;
  // The array keeps whatever the previous call left: counters and status must start at zero.
  MKB_CUDA(cudaMemsetAsync(words, 0, (size_t)SW_FLAGS * 4, static_cast<cudaStream_t>(stream)));
  mk_symm_view sv, cv;
  memset(&sv, 0, sizeof(sv));
  memset(&cv, 0, sizeof(cv));
  sv.rank = 0; sv.world = 1; sv.bytes = (size_t)kNoAllocSyncWords * 4; sv.peer[0] = words;
  cv.rank = 0; cv.world = 1; cv.bytes = (size_t)M * N * 2; cv.peer[0] = C;
  OpArgs a;
  memset(&a, 0, sizeof(a));
  a.op = OP_RS; a.A = A; a.a_rows = M; a.B = B; a.C = C;
  a.M = M; a.N = N; a.K = K; a.b_layout = MK_B_NK; a.rank = 0; a.world = 1;
  a.sync = &sv; a.data = &cv;
  return run_op(a, static_cast<cudaStream_t>(stream));
}

int mk_gemm_ar_launch(const void* A, const void* B, const mk_symm_view* C,
                      const mk_symm_view* barrier, const mk_symm_view* C_final, int M, int N,
                      int K, uint32_t epoch, int b_layout, void* stream) {
  if (!A || !B) return set_error(MK_ERR_INVALID, "mk_gemm_ar_launch: null operand");
  if (M < 1 || N < 1) return set_error(MK_ERR_INVALID, "mk_gemm_ar_launch: bad shape");
  if (b_layout != MK_B_KN && b_layout != MK_B_NK)
    return set_error(MK_ERR_INVALID, "mk_gemm_ar_launch: unknown B layout %d", b_layout);
  int rc = check_view(C, "C", (size_t)M * N * 2);
  if (rc != MK_OK) return rc;
  rc = check_view(C_final, "C_final", (size_t)M * N * 2);
  if (rc != MK_OK) return rc;
  rc = check_view(barrier, "barrier", (size_t)SW_FLAGS * 4);
  if (rc != MK_OK) return rc;
  if (C->world != barrier->world || C->rank != barrier->rank || C_final->world != C->world ||
      C_final->rank != C->rank)
    return set_error(MK_ERR_INVALID, "C, C_final and barrier disagree on rank/world");
  OpArgs a;
  memset(&a, 0, sizeof(a));
  a.op = OP_AR; a.A = A; a.a_rows = M; a.B = B;
  a.M = M; a.N = N; a.K = K; a.b_layout = b_layout; a.rank = C->rank; a.world = C->world;
  a.sync = barrier; a.data = C; a.out = C_final; a.epoch = epoch;
  a.C = C->peer[C->rank];
  return run_op(a, static_cast<cudaStream_t>(stream));
}

int mk_op_status(const mk_symm_view* sync, uint32_t out4[4]) {
  int rc = check_view(sync, "sync", (size_t)SW_FLAGS * 4);
  if (rc != MK_OK) return rc;
  uint32_t w[4] = {0, 0, 0, 0};
  MKB_CUDA(cudaMemcpy(w, static_cast<uint32_t*>(sync->peer[sync->rank]) + SW_STATUS, sizeof(w),
                      cudaMemcpyDeviceToHost));
  if (out4) memcpy(out4, w, sizeof(w));
  if (w[0] != 0)
    return set_error(MK_ERR_DEVICE_WAIT,
                     "device wait expired: code=%u cta=%u role=%u detail=(%u,%u)", w[0], w[1] >> 8,
                     w[1] & 255u, w[2], w[3]);
  return MK_OK;
}

int mk_op_status_clear(const mk_symm_view* sync, void* stream) {
  int rc = check_view(sync, "sync", (size_t)SW_FLAGS * 4);
  if (rc != MK_OK) return rc;
  MKB_CUDA(cudaMemsetAsync(static_cast<uint32_t*>(sync->peer[sync->rank]) + SW_STATUS, 0, 16,
                           static_cast<cudaStream_t>(stream)));
  return MK_OK;
}

int mk_plan_op(int op, int rank, int world, int M, int N, int K, int b_layout, int num_sms,
               mk_plan* out) {
  if (!out) return set_error(MK_ERR_INVALID, "mk_plan_op: null out");
  Plan pl;
  int rc = make_plan(options_snapshot(), op, rank, world, M, N, K, b_layout, num_sms, &pl);
  if (rc != MK_OK) return rc;
  out->block_n = pl.sched.block_n;
  out->stages = pl.stages;
  out->n_comm = pl.n_comm;
  out->grid = pl.grid;
  out->smem_bytes = pl.smem;
  out->row_blocks = pl.sched.P;
  out->col_blocks = pl.sched.Q;
  out->k_blocks = pl.k_blocks;
  out->part_rows = pl.sched.part_rows;
  out->part_blocks = pl.sched.part_blocks;
  out->interleave = pl.sched.interleave;
  out->group_rows = pl.sched.group_rows;
  out->sync_words = sync_words_needed(pl.sched);
  out->group_cols = pl.sched.group_cols;
  return MK_OK;
}

int mk_sched_tiles(int op, int rank, int world, int M, int N, int block_n, int group_rows,
                   int group_cols, int* row0, int* rows, int* col0, int* rowblock, int cap) {
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || block_n < 8 || M < 1 || N < 1)
    return set_error(MK_ERR_INVALID, "mk_sched_tiles: bad arguments");
  const Sched s = make_sched(op, rank, world, M, N, block_n, group_rows, group_cols);
  const int total = s.P * s.Q;
  for (int t = 0; t < total && t < cap; ++t) {
    int rb, q;
    tile_to_coord(s, t, &rb, &q);
    if (row0) row0[t] = rowblock_row0(s, rb);
    if (rows) rows[t] = rowblock_rows(s, rb);
    if (col0) col0[t] = q * block_n;
    if (rowblock) rowblock[t] = rb;
  }
  return total;
}

int mk_sched_work_items(int total_tiles, int n_comp, int cg, int k_blocks, int max_parts, int cta,
                        int* tile, int* kb0, int* kb1, int* piece, int cap) {
  if (total_tiles < 1 || n_comp < 1 || (cg != 1 && cg != 2) || n_comp % cg != 0 ||
      total_tiles % cg != 0 || k_blocks < 1 || cta < 0 || cta >= n_comp)
    return set_error(MK_ERR_INVALID, "mk_sched_work_items: bad arguments");
  const SplitPlan sp = plan_split(total_tiles, n_comp, cg, k_blocks, max_parts);
  int n = 0;
  WorkItem w;
  for (int it = 0; cta_work_item(sp, total_tiles, n_comp, cg, k_blocks, cta, it, &w); ++it) {
    if (n < cap) {
      if (tile) tile[n] = w.t;
      if (kb0) kb0[n] = w.kb0;
      if (kb1) kb1[n] = w.kb1;
      if (piece) piece[n] = w.piece;
    }
    ++n;
  }
  return n;
}

int mk_sched_owner_items(int op, int world, int M, int N, int block_n, int owner, int* row0,
                         int* row1, int cap) {
  if (world < 1 || world > kMaxWorld || owner < 0 || owner >= world || M < 1 || N < 1 ||
      block_n < 8)
    return set_error(MK_ERR_INVALID, "mk_sched_owner_items: bad arguments");
  const Sched s = make_sched(op, owner, world, M, N, block_n, 8);
  const int n = owner_num_items(s, owner);
  for (int k = 0; k < n && k < cap; ++k) {
    int a, b;
    owner_item_rows(s, owner, k, &a, &b);
    if (row0) row0[k] = a;
    if (row1) row1[k] = b;
  }
  return n;
}

}  // extern "C"
