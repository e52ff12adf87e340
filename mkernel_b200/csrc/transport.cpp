// Intra-node transport for one NVSwitch box: rank rendezvous, file-descriptor exchange, and
// symmetric device allocations (CUDA virtual memory management + optional NVSwitch multicast).
//
// What it replaces in the reference (behaviour, not code):
//   include/comm/local_broker.cuh:362-534  shm segment + rank-0 hub + /tmp unix sockets
//   include/comm/ipc.cuh:100-122           POSIX-fd import of peer allocations
//   include/comm/vmm.cuh:29-119            cuMemCreate / map / multicast bind
//   include/dist/parallel_buffer.cuh:87-338  ParallelBuffer construction sequence
// Design here: no hub and nothing on the file system.  Every rank binds one datagram socket in
// the Linux abstract namespace (it disappears with the process, so there is no stale state to
// reclaim) and collectives are all-to-all datagram exchanges driven by a progress loop that
// keeps receiving while it retries sends, so no ordering of ranks can deadlock.  Descriptors
// travel as SCM_RIGHTS ancillary data.  Every blocking step has a deadline.
#include <cuda.h>
#include <cuda_runtime_api.h>
#include <errno.h>
#include <poll.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <deque>
#include <string>
#include <vector>

#include "../../include/mkernel_b200.h"
#include "host_util.h"

namespace mkb {

// ------------------------------------------------------------------------------------------
// error text + driver entry points
// ------------------------------------------------------------------------------------------
static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int driver_entry(const char* symbol, void** fn) {
  cudaDriverEntryPointQueryResult q;
  void* p = nullptr;
  cudaError_t e = cudaGetDriverEntryPoint(symbol, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
    (void)cudaGetLastError();
    return set_error(MK_ERR_CUDA, "driver entry point %s unavailable (%s)", symbol,
                     e != cudaSuccess ? cudaGetErrorString(e) : "not found");
  }
  *fn = p;
  return MK_OK;
}

static double now_s() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec + 1e-9 * ts.tv_nsec;
}

// ------------------------------------------------------------------------------------------
// datagram rendezvous
// ------------------------------------------------------------------------------------------
enum MsgKind : uint32_t { MSG_BYTES = 1, MSG_FD = 2 };
constexpr uint32_t kMagic = 0x6d6b6232u;  // "mkb2"
constexpr size_t kMaxPayload = 256;

struct MsgHeader {
  uint32_t magic, kind, seq, src, len;
};
struct Msg {
  MsgHeader h;
  unsigned char payload[kMaxPayload];
  int fd;
};

}  // namespace mkb

struct mk_comm {
  int rank = 0, world = 1, device = 0;
  int sock = -1;
  uint32_t seq = 0;
  double timeout_s = 120.0;
  std::string key;
  std::deque<mkb::Msg> stash;
};

namespace mkb {

// Abstract-namespace address "mkb200/<key>/<rank>".  A key that would not fit (a fully
// qualified host name plus a run id, say) is replaced by two 64-bit hashes of it, so that the
// rank suffix is never cut off and two long keys sharing a prefix do not collide.
static socklen_t make_addr(const std::string& key, int rank, sockaddr_un* a) {
  memset(a, 0, sizeof(*a));
  a->sun_family = AF_UNIX;
  char name[100];
  int n;
  if (key.size() <= 64) {
    n = snprintf(name, sizeof(name), "mkb200/%s/%d", key.c_str(), rank);
  } else {
    uint64_t h1 = 1469598103934665603ull, h2 = 0x9E3779B97F4A7C15ull;
    for (unsigned char ch : key) {
      h1 = (h1 ^ ch) * 1099511628211ull;                    // FNV-1a
      h2 = (h2 + ch) * 0xFF51AFD7ED558CCDull; h2 ^= h2 >> 33;
    }
    n = snprintf(name, sizeof(name), "mkb200/#%016llx%016llx.%zu/%d", (unsigned long long)h1,
                 (unsigned long long)h2, key.size(), rank);
  }
  if (n < 0) n = 0;
  if (n > (int)sizeof(name) - 1) n = sizeof(name) - 1;      // never read past `name`
  if (n > (int)sizeof(a->sun_path) - 2) n = sizeof(a->sun_path) - 2;
  a->sun_path[0] = '\0';  // abstract namespace
  memcpy(a->sun_path + 1, name, n);
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

// Non-blocking send of one message (optionally carrying a descriptor).  1 = sent, 0 = retry later.
static int try_send(mk_comm* c, int dst, const Msg& m) {
  sockaddr_un addr;
  socklen_t alen = make_addr(c->key, dst, &addr);
  unsigned char buf[sizeof(MsgHeader) + kMaxPayload];
  memcpy(buf, &m.h, sizeof(MsgHeader));
  memcpy(buf + sizeof(MsgHeader), m.payload, m.h.len);
  iovec iov{buf, sizeof(MsgHeader) + m.h.len};
  msghdr mh;
  memset(&mh, 0, sizeof(mh));
  mh.msg_name = &addr;
  mh.msg_namelen = alen;
  mh.msg_iov = &iov;
  mh.msg_iovlen = 1;
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  if (m.h.kind == MSG_FD) {
    memset(ctrl, 0, sizeof(ctrl));
    mh.msg_control = ctrl;
    mh.msg_controllen = sizeof(ctrl);
    cmsghdr* cm = CMSG_FIRSTHDR(&mh);
    cm->cmsg_level = SOL_SOCKET;
    cm->cmsg_type = SCM_RIGHTS;
    cm->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(cm), &m.fd, sizeof(int));
  }
  ssize_t r = sendmsg(c->sock, &mh, MSG_DONTWAIT | MSG_NOSIGNAL);
  if (r >= 0) return 1;
  if (errno == EAGAIN || errno == EWOULDBLOCK || errno == ECONNREFUSED || errno == ENOENT ||
      errno == ENOBUFS || errno == EINTR || errno == ENOTCONN)
    return 0;  // peer not bound yet or its queue is full
  return set_error(MK_ERR_TRANSPORT, "sendmsg to rank %d failed: %s", dst, strerror(errno));
}

// Drains whatever is readable (waits at most wait_ms for the first datagram) into the stash.
static int pump(mk_comm* c, int wait_ms) {
  pollfd pfd{c->sock, POLLIN, 0};
  int pr = poll(&pfd, 1, wait_ms);
  if (pr < 0 && errno != EINTR)
    return set_error(MK_ERR_TRANSPORT, "poll failed: %s", strerror(errno));
  while (true) {
    unsigned char buf[sizeof(MsgHeader) + kMaxPayload];
    iovec iov{buf, sizeof(buf)};
    msghdr mh;
    memset(&mh, 0, sizeof(mh));
    mh.msg_iov = &iov;
    mh.msg_iovlen = 1;
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
    mh.msg_control = ctrl;
    mh.msg_controllen = sizeof(ctrl);
    ssize_t r = recvmsg(c->sock, &mh, MSG_DONTWAIT | MSG_CMSG_CLOEXEC);
    if (r < 0) {
      if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) return MK_OK;
      return set_error(MK_ERR_TRANSPORT, "recvmsg failed: %s", strerror(errno));
    }
    Msg m;
    memset(&m, 0, sizeof(m));
    m.fd = -1;
    for (cmsghdr* cm = CMSG_FIRSTHDR(&mh); cm; cm = CMSG_NXTHDR(&mh, cm)) {
      if (cm->cmsg_level == SOL_SOCKET && cm->cmsg_type == SCM_RIGHTS)
        memcpy(&m.fd, CMSG_DATA(cm), sizeof(int));
    }
    if ((size_t)r < sizeof(MsgHeader)) { if (m.fd >= 0) close(m.fd); continue; }
    memcpy(&m.h, buf, sizeof(MsgHeader));
    if (m.h.magic != kMagic || m.h.len > kMaxPayload || (size_t)r != sizeof(MsgHeader) + m.h.len ||
        m.h.src >= (uint32_t)c->world) {
      if (m.fd >= 0) close(m.fd);
      continue;  // not one of ours
    }
    memcpy(m.payload, buf + sizeof(MsgHeader), m.h.len);
    c->stash.push_back(m);
  }
}

// All-to-all exchange of one message per peer for sequence number `seq`.
// out[r] receives rank r's message (out[rank] is not touched).
static int exchange(mk_comm* c, uint32_t kind, const void* payload, size_t len, int fd,
                    std::vector<Msg>* out) {
  if (len > kMaxPayload) return set_error(MK_ERR_INVALID, "payload of %zu bytes exceeds %zu", len, kMaxPayload);
  const uint32_t seq = ++c->seq;
  out->assign(c->world, Msg());
  std::vector<char> sent(c->world, 0), got(c->world, 0);
  sent[c->rank] = got[c->rank] = 1;
  Msg mine;
  memset(&mine, 0, sizeof(mine));
  mine.h = MsgHeader{kMagic, kind, seq, (uint32_t)c->rank, (uint32_t)len};
  if (len) memcpy(mine.payload, payload, len);
  mine.fd = fd;
  const double deadline = now_s() + c->timeout_s;
  int n_sent = 1, n_got = 1;
  while (n_sent < c->world || n_got < c->world) {
    bool progressed = false;
    for (int r = 0; r < c->world; ++r) {
      if (sent[r]) continue;
      int s = try_send(c, r, mine);
      if (s < 0) return s;
      if (s == 1) { sent[r] = 1; ++n_sent; progressed = true; }
    }
    int rc = pump(c, progressed ? 0 : 2);
    if (rc != MK_OK) return rc;
    for (auto it = c->stash.begin(); it != c->stash.end();) {
      if (it->h.seq == seq && it->h.kind == kind && !got[it->h.src]) {
        (*out)[it->h.src] = *it;
        got[it->h.src] = 1;
        ++n_got;
        it = c->stash.erase(it);
      } else {
        ++it;
      }
    }
    if (now_s() > deadline) {
      int missing = -1;
      for (int r = 0; r < c->world; ++r) if (!got[r] || !sent[r]) { missing = r; break; }
      for (auto& m : *out) if (m.h.magic == kMagic && m.fd >= 0) close(m.fd);
      return set_error(MK_ERR_TRANSPORT, "rendezvous step %u timed out after %.0f s waiting for rank %d",
                       seq, c->timeout_s, missing);
    }
  }
  return MK_OK;
}

// ------------------------------------------------------------------------------------------
// driver API (looked up lazily; the library does not link libcuda)
// ------------------------------------------------------------------------------------------
struct Driver {
  bool ready = false;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MemExport)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*MemImport)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*MemGetGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*McCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*McAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*McBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
  CUresult (*McUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*McGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
  CUresult (*DeviceGet)(CUdevice*, int);
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  CUresult (*GetErrorString)(CUresult, const char**);
};
static Driver g_drv;

static int load_driver() {
  if (g_drv.ready) return MK_OK;
#define MKB_SYM(field, name)                                         \
  do {                                                               \
    void* p_ = nullptr;                                              \
    int rc_ = driver_entry(name, &p_);                               \
    if (rc_ != MK_OK) return rc_;                                    \
    g_drv.field = reinterpret_cast<decltype(g_drv.field)>(p_);       \
  } while (0)
  MKB_SYM(MemCreate, "cuMemCreate");
  MKB_SYM(MemRelease, "cuMemRelease");
  MKB_SYM(MemAddressReserve, "cuMemAddressReserve");
  MKB_SYM(MemAddressFree, "cuMemAddressFree");
  MKB_SYM(MemMap, "cuMemMap");
  MKB_SYM(MemUnmap, "cuMemUnmap");
  MKB_SYM(MemSetAccess, "cuMemSetAccess");
  MKB_SYM(MemExport, "cuMemExportToShareableHandle");
  MKB_SYM(MemImport, "cuMemImportFromShareableHandle");
  MKB_SYM(MemGetGranularity, "cuMemGetAllocationGranularity");
  MKB_SYM(McCreate, "cuMulticastCreate");
  MKB_SYM(McAddDevice, "cuMulticastAddDevice");
  MKB_SYM(McBindMem, "cuMulticastBindMem");
  MKB_SYM(McUnbind, "cuMulticastUnbind");
  MKB_SYM(McGetGranularity, "cuMulticastGetGranularity");
  MKB_SYM(DeviceGet, "cuDeviceGet");
  MKB_SYM(DeviceGetAttribute, "cuDeviceGetAttribute");
  MKB_SYM(GetErrorString, "cuGetErrorString");
#undef MKB_SYM
  g_drv.ready = true;
  return MK_OK;
}

static int drv_fail(const char* what, CUresult r) {
  const char* s = nullptr;
  if (g_drv.GetErrorString) g_drv.GetErrorString(r, &s);
  return set_error(MK_ERR_CUDA, "%s failed: %s (CUresult %d)", what, s ? s : "?", (int)r);
}
#define MKB_DRV(call, what)                          \
  do {                                               \
    CUresult r_ = (call);                            \
    if (r_ != CUDA_SUCCESS) return drv_fail(what, r_); \
  } while (0)

}  // namespace mkb

struct mk_symm {
  mk_comm* comm = nullptr;
  size_t bytes = 0;        // requested
  size_t mapped = 0;       // granularity-rounded
  CUmemGenericAllocationHandle local_handle = 0;
  CUmemGenericAllocationHandle peer_handle[MK_MAX_WORLD] = {};
  CUdeviceptr va[MK_MAX_WORLD] = {};
  CUmemGenericAllocationHandle mc_handle = 0;
  CUdeviceptr mc_va = 0;
  bool mc_bound = false;
};

using namespace mkb;

static int map_handle(CUmemGenericAllocationHandle h, size_t size, size_t gran, int device,
                      CUdeviceptr* va) {
  MKB_DRV(g_drv.MemAddressReserve(va, size, gran, 0, 0), "cuMemAddressReserve");
  MKB_DRV(g_drv.MemMap(*va, size, 0, h, 0), "cuMemMap");
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  MKB_DRV(g_drv.MemSetAccess(*va, size, &acc, 1), "cuMemSetAccess");
  return MK_OK;
}

extern "C" {

const char* mk_last_error(void) { return g_err; }

int mk_comm_create(const char* key, int rank, int world, int device, mk_comm** out) {
  if (!out) return set_error(MK_ERR_INVALID, "mk_comm_create: null out");
  if (world < 1 || world > MK_MAX_WORLD || rank < 0 || rank >= world)
    return set_error(MK_ERR_INVALID, "mk_comm_create: rank=%d world=%d out of range (world <= %d)",
                     rank, world, MK_MAX_WORLD);
  mk_comm* c = new mk_comm();
  c->rank = rank;
  c->world = world;
  c->device = device;
  c->key = key ? key : "default";
  if (const char* t = getenv("MKB200_RENDEZVOUS_TIMEOUT_S")) {
    double v = atof(t);
    if (v > 0) c->timeout_s = v;
  }
  if (world > 1) {
    c->sock = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
    if (c->sock < 0) {
      int e = errno;
      delete c;
      return set_error(MK_ERR_TRANSPORT, "socket failed: %s", strerror(e));
    }
    sockaddr_un addr;
    socklen_t alen = make_addr(c->key, rank, &addr);
    if (bind(c->sock, reinterpret_cast<sockaddr*>(&addr), alen) != 0) {
      int e = errno;
      close(c->sock);
      delete c;
      return set_error(MK_ERR_TRANSPORT, "bind of rendezvous name for key '%s' rank %d failed: %s",
                       key ? key : "default", rank, strerror(e));
    }
  }
  *out = c;
  return MK_OK;
}

int mk_comm_destroy(mk_comm* c) {
  if (!c) return MK_OK;
  for (auto& m : c->stash) if (m.fd >= 0) close(m.fd);
  if (c->sock >= 0) close(c->sock);
  delete c;
  return MK_OK;
}

int mk_comm_rank(const mk_comm* c) { return c ? c->rank : -1; }
int mk_comm_world(const mk_comm* c) { return c ? c->world : -1; }

int mk_comm_allgather(mk_comm* c, const void* in, size_t bytes, void* out) {
  if (!c || (!in && bytes) || !out) return set_error(MK_ERR_INVALID, "mk_comm_allgather: null argument");
  if (bytes > kMaxPayload) return set_error(MK_ERR_INVALID, "mk_comm_allgather: at most %zu bytes per rank", kMaxPayload);
  unsigned char* o = static_cast<unsigned char*>(out);
  if (bytes) memcpy(o + (size_t)c->rank * bytes, in, bytes);
  if (c->world == 1) return MK_OK;
  std::vector<Msg> msgs;
  int rc = exchange(c, MSG_BYTES, in, bytes, -1, &msgs);
  if (rc != MK_OK) return rc;
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    if (msgs[r].h.len != bytes)
      return set_error(MK_ERR_TRANSPORT, "rank %d contributed %u bytes, expected %zu", r, msgs[r].h.len, bytes);
    if (bytes) memcpy(o + (size_t)r * bytes, msgs[r].payload, bytes);
  }
  return MK_OK;
}

int mk_comm_barrier(mk_comm* c) {
  if (!c) return set_error(MK_ERR_INVALID, "mk_comm_barrier: null comm");
  unsigned char token = 1, all[MK_MAX_WORLD];
  return mk_comm_allgather(c, &token, 1, all);
}

int mk_comm_allgather_fd(mk_comm* c, int fd, int* out_fds) {
  if (!c || !out_fds || fd < 0) return set_error(MK_ERR_INVALID, "mk_comm_allgather_fd: bad argument");
  for (int r = 0; r < c->world; ++r) out_fds[r] = -1;
  out_fds[c->rank] = dup(fd);
  if (out_fds[c->rank] < 0) return set_error(MK_ERR_TRANSPORT, "dup failed: %s", strerror(errno));
  if (c->world == 1) return MK_OK;
  std::vector<Msg> msgs;
  int rc = exchange(c, MSG_FD, nullptr, 0, fd, &msgs);
  if (rc != MK_OK) { close(out_fds[c->rank]); out_fds[c->rank] = -1; return rc; }
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    if (msgs[r].fd < 0) {
      for (int q = 0; q < c->world; ++q) {
        if (q != c->rank && msgs[q].fd >= 0) close(msgs[q].fd);
      }
      close(out_fds[c->rank]);
      for (int q = 0; q < c->world; ++q) out_fds[q] = -1;
      return set_error(MK_ERR_TRANSPORT, "rank %d sent no descriptor", r);
    }
    out_fds[r] = msgs[r].fd;
  }
  return MK_OK;
}

// ------------------------------------------------------------------------------------------
// symmetric allocations
// ------------------------------------------------------------------------------------------
int mk_symm_free(mk_symm* b) {
  if (!b) return MK_OK;
  if (g_drv.ready) {
    if (b->mc_va) {
      g_drv.MemUnmap(b->mc_va, b->mapped);
      g_drv.MemAddressFree(b->mc_va, b->mapped);
    }
    if (b->mc_bound) {
      CUdevice dev;
      if (g_drv.DeviceGet(&dev, b->comm->device) == CUDA_SUCCESS)
        g_drv.McUnbind(b->mc_handle, dev, 0, b->mapped);
    }
    if (b->mc_handle) g_drv.MemRelease(b->mc_handle);
    const int world = b->comm ? b->comm->world : 1;
    const int rank = b->comm ? b->comm->rank : 0;
    for (int r = 0; r < world; ++r) {
      if (b->va[r]) {
        g_drv.MemUnmap(b->va[r], b->mapped);
        g_drv.MemAddressFree(b->va[r], b->mapped);
      }
      if (r != rank && b->peer_handle[r]) g_drv.MemRelease(b->peer_handle[r]);
    }
    if (b->local_handle) g_drv.MemRelease(b->local_handle);
  }
  delete b;
  return MK_OK;
}

int mk_symm_alloc(mk_comm* c, size_t bytes, int want_multicast, mk_symm** out) {
  if (!c || !out) return set_error(MK_ERR_INVALID, "mk_symm_alloc: null argument");
  if (bytes == 0) return set_error(MK_ERR_INVALID, "mk_symm_alloc: zero bytes");
  int rc = load_driver();
  if (rc != MK_OK) return rc;
  MKB_CUDA(cudaSetDevice(c->device));
  MKB_CUDA(cudaFree(0));  // make sure the primary context exists

  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = c->device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  MKB_DRV(g_drv.MemGetGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
          "cuMemGetAllocationGranularity");

  // Multicast needs every rank to agree; a rank that cannot do it vetoes for all.
  int use_mc = (want_multicast && c->world > 1) ? 1 : 0;
  CUmulticastObjectProp mcprop;
  memset(&mcprop, 0, sizeof(mcprop));
  if (use_mc) {
    CUdevice dev;
    MKB_DRV(g_drv.DeviceGet(&dev, c->device), "cuDeviceGet");
    int supported = 0;
    if (g_drv.DeviceGetAttribute(&supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS)
      supported = 0;
    if (!supported) use_mc = 0;
  }
  if (want_multicast && c->world > 1) {
    unsigned char mine = (unsigned char)use_mc, all[MK_MAX_WORLD];
    rc = mk_comm_allgather(c, &mine, 1, all);
    if (rc != MK_OK) return rc;
    for (int r = 0; r < c->world; ++r) if (!all[r]) use_mc = 0;
  }
  if (use_mc) {
    mcprop.numDevices = c->world;
    mcprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mcprop.flags = 0;
    mcprop.size = bytes;  // provisional, only the granularity is needed here
    size_t mc_gran = 0;
    MKB_DRV(g_drv.McGetGranularity(&mc_gran, &mcprop, CU_MULTICAST_GRANULARITY_RECOMMENDED),
            "cuMulticastGetGranularity");
    if (mc_gran > gran) gran = mc_gran;
  }
  const size_t mapped = (bytes + gran - 1) / gran * gran;

  mk_symm* b = new mk_symm();
  b->comm = c;
  b->bytes = bytes;
  b->mapped = mapped;
#define MKB_FAIL_IF(expr, what)                  \
  do {                                           \
    CUresult r_ = (expr);                        \
    if (r_ != CUDA_SUCCESS) {                    \
      int code_ = drv_fail(what, r_);            \
      mk_symm_free(b);                           \
      return code_;                              \
    }                                            \
  } while (0)

  MKB_FAIL_IF(g_drv.MemCreate(&b->local_handle, mapped, &prop, 0), "cuMemCreate");
  b->peer_handle[c->rank] = b->local_handle;
  rc = map_handle(b->local_handle, mapped, gran, c->device, &b->va[c->rank]);
  if (rc != MK_OK) { mk_symm_free(b); return rc; }

  if (c->world > 1) {
    int fd = -1;
    MKB_FAIL_IF(g_drv.MemExport(&fd, b->local_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
                "cuMemExportToShareableHandle");
    int fds[MK_MAX_WORLD];
    rc = mk_comm_allgather_fd(c, fd, fds);
    close(fd);
    if (rc != MK_OK) { mk_symm_free(b); return rc; }
    for (int r = 0; r < c->world; ++r) {
      if (r == c->rank) { close(fds[r]); continue; }
      CUresult ir = g_drv.MemImport(&b->peer_handle[r], (void*)(uintptr_t)fds[r],
                                    CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      close(fds[r]);
      if (ir != CUDA_SUCCESS) {
        for (int q = r + 1; q < c->world; ++q) if (q != c->rank) close(fds[q]);
        int code = drv_fail("cuMemImportFromShareableHandle", ir);
        mk_symm_free(b);
        return code;
      }
      rc = map_handle(b->peer_handle[r], mapped, gran, c->device, &b->va[r]);
      if (rc != MK_OK) {
        for (int q = r + 1; q < c->world; ++q) if (q != c->rank) close(fds[q]);
        mk_symm_free(b);
        return rc;
      }
    }
  }

  if (use_mc) {
    // Rank 0 creates the multicast object and shares it; everyone adds its device, then (after
    // all devices are in) binds its own allocation and maps the multicast address.
    mcprop.size = mapped;
    int mfd = -1;
    if (c->rank == 0) {
      MKB_FAIL_IF(g_drv.McCreate(&b->mc_handle, &mcprop), "cuMulticastCreate");
      MKB_FAIL_IF(g_drv.MemExport(&mfd, b->mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
                  "cuMemExportToShareableHandle(multicast)");
    } else {
      mfd = dup(c->sock);  // placeholder descriptor so that every rank contributes one
    }
    int fds[MK_MAX_WORLD];
    rc = mk_comm_allgather_fd(c, mfd, fds);
    if (mfd >= 0) close(mfd);
    if (rc != MK_OK) { mk_symm_free(b); return rc; }
    if (c->rank != 0) {
      CUresult ir = g_drv.MemImport(&b->mc_handle, (void*)(uintptr_t)fds[0],
                                    CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      for (int r = 0; r < c->world; ++r) close(fds[r]);
      if (ir != CUDA_SUCCESS) {
        int code = drv_fail("cuMemImportFromShareableHandle(multicast)", ir);
        mk_symm_free(b);
        return code;
      }
    } else {
      for (int r = 0; r < c->world; ++r) close(fds[r]);
    }
    CUdevice dev;
    MKB_FAIL_IF(g_drv.DeviceGet(&dev, c->device), "cuDeviceGet");
    MKB_FAIL_IF(g_drv.McAddDevice(b->mc_handle, dev), "cuMulticastAddDevice");
    rc = mk_comm_barrier(c);
    if (rc != MK_OK) { mk_symm_free(b); return rc; }
    MKB_FAIL_IF(g_drv.McBindMem(b->mc_handle, 0, b->local_handle, 0, mapped, 0), "cuMulticastBindMem");
    b->mc_bound = true;
    rc = map_handle(b->mc_handle, mapped, gran, c->device, &b->mc_va);
    if (rc != MK_OK) { mk_symm_free(b); return rc; }
  }
#undef MKB_FAIL_IF

  // Nobody may touch a peer mapping before every rank has finished mapping.
  rc = mk_comm_barrier(c);
  if (rc != MK_OK) { mk_symm_free(b); return rc; }
  *out = b;
  return MK_OK;
}

int mk_symm_get_view(const mk_symm* b, mk_symm_view* out) {
  if (!b || !out) return set_error(MK_ERR_INVALID, "mk_symm_get_view: null argument");
  memset(out, 0, sizeof(*out));
  out->rank = b->comm->rank;
  out->world = b->comm->world;
  out->bytes = b->bytes;
  for (int r = 0; r < b->comm->world; ++r) out->peer[r] = reinterpret_cast<void*>(b->va[r]);
  out->mc = reinterpret_cast<void*>(b->mc_va);
  return MK_OK;
}

}  // extern "C"
