// Symmetric regions with an NVSwitch multicast alias, built with the CUDA driver's virtual memory
// API: cuMemCreate per GPU, every GPU's memory mapped on every GPU (peer stores and loads), and one
// multicast object (cuMulticastCreate / AddDevice / BindMem) whose mapping takes multimem
// instructions: a store to it lands in all bound memories, a ld_reduce returns their sum.
//
// Two set-ups behind the same handle:
//   hc_mc_create_local   one process drives all GPUs (a thread per GPU): no handle leaves the process;
//   hc_mc_create_shared  one process per GPU: memory and multicast handles travel as POSIX file
//                        descriptors over a unix-domain socket (SCM_RIGHTS), rank 0 acting as the hub.
// The reference has no counterpart: its bytes travel through MPI (HomComp/src/cuda_awareallreduce.cu:208-255).
//
// Only multimem instructions and ordinary loads / stores ever touch these mappings; no TMA copy is
// issued on them.  Every rank must leave together (hc_mc_destroy after a barrier of the caller's): a
// rank that dies while its memory is bound to the multicast object can disturb the others' GPUs.
#include <cuda.h>
#include <cuda_runtime.h>
#include <errno.h>
#include <stdio.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <sys/un.h>
#include <unistd.h>

#include <new>
#include <vector>

#include "hc_format.h"
#include "homcomp_b200.h"

namespace {

// driver entry points, looked up through the runtime so that the library needs no link against libcuda
template <typename F>
F driver_fn(const char* name) {
  void* f = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) f = nullptr;
  return reinterpret_cast<F>(f);
}
#define HC_DRV(name) static auto p_##name = driver_fn<decltype(&name)>(#name)

struct Driver {
  decltype(&cuDeviceGet) DeviceGet;
  decltype(&cuDeviceGetAttribute) DeviceGetAttribute;
  decltype(&cuMemCreate) MemCreate;
  decltype(&cuMemRelease) MemRelease;
  decltype(&cuMemAddressReserve) MemAddressReserve;
  decltype(&cuMemAddressFree) MemAddressFree;
  decltype(&cuMemMap) MemMap;
  decltype(&cuMemUnmap) MemUnmap;
  decltype(&cuMemSetAccess) MemSetAccess;
  decltype(&cuMemGetAllocationGranularity) MemGetAllocationGranularity;
  decltype(&cuMemExportToShareableHandle) MemExportToShareableHandle;
  decltype(&cuMemImportFromShareableHandle) MemImportFromShareableHandle;
  decltype(&cuMulticastCreate) MulticastCreate;
  decltype(&cuMulticastAddDevice) MulticastAddDevice;
  decltype(&cuMulticastBindMem) MulticastBindMem;
  decltype(&cuMulticastUnbind) MulticastUnbind;
  decltype(&cuMulticastGetGranularity) MulticastGetGranularity;
  bool ok = false;
};
const Driver& drv() {
  static Driver d = [] {
    Driver x;
    x.DeviceGet = driver_fn<decltype(&cuDeviceGet)>("cuDeviceGet");
    x.DeviceGetAttribute = driver_fn<decltype(&cuDeviceGetAttribute)>("cuDeviceGetAttribute");
    x.MemCreate = driver_fn<decltype(&cuMemCreate)>("cuMemCreate");
    x.MemRelease = driver_fn<decltype(&cuMemRelease)>("cuMemRelease");
    x.MemAddressReserve = driver_fn<decltype(&cuMemAddressReserve)>("cuMemAddressReserve");
    x.MemAddressFree = driver_fn<decltype(&cuMemAddressFree)>("cuMemAddressFree");
    x.MemMap = driver_fn<decltype(&cuMemMap)>("cuMemMap");
    x.MemUnmap = driver_fn<decltype(&cuMemUnmap)>("cuMemUnmap");
    x.MemSetAccess = driver_fn<decltype(&cuMemSetAccess)>("cuMemSetAccess");
    x.MemGetAllocationGranularity = driver_fn<decltype(&cuMemGetAllocationGranularity)>("cuMemGetAllocationGranularity");
    x.MemExportToShareableHandle = driver_fn<decltype(&cuMemExportToShareableHandle)>("cuMemExportToShareableHandle");
    x.MemImportFromShareableHandle = driver_fn<decltype(&cuMemImportFromShareableHandle)>("cuMemImportFromShareableHandle");
    x.MulticastCreate = driver_fn<decltype(&cuMulticastCreate)>("cuMulticastCreate");
    x.MulticastAddDevice = driver_fn<decltype(&cuMulticastAddDevice)>("cuMulticastAddDevice");
    x.MulticastBindMem = driver_fn<decltype(&cuMulticastBindMem)>("cuMulticastBindMem");
    x.MulticastUnbind = driver_fn<decltype(&cuMulticastUnbind)>("cuMulticastUnbind");
    x.MulticastGetGranularity = driver_fn<decltype(&cuMulticastGetGranularity)>("cuMulticastGetGranularity");
    x.ok = x.DeviceGet && x.DeviceGetAttribute && x.MemCreate && x.MemRelease && x.MemAddressReserve && x.MemAddressFree &&
           x.MemMap && x.MemUnmap && x.MemSetAccess && x.MemGetAllocationGranularity && x.MemExportToShareableHandle &&
           x.MemImportFromShareableHandle && x.MulticastCreate && x.MulticastAddDevice && x.MulticastBindMem &&
           x.MulticastUnbind && x.MulticastGetGranularity;
    return x;
  }();
  return d;
}

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

struct hc_mc_region {
  int n = 0;            // GPUs (ranks) that share the object
  int own = -1;         // shared set-up: this process's rank (it owns mem[own] and its device); local: -1
  size_t size = 0;      // mapped bytes (the request rounded up to the multicast granularity)
  bool has_mc = false;
  CUmemGenericAllocationHandle mc = 0;
  std::vector<CUmemGenericAllocationHandle> mem;  // one per GPU (imported handles in the shared set-up)
  std::vector<CUdeviceptr> uc;                    // unicast mapping of every GPU's memory
  CUdeviceptr mc_va = 0;
  std::vector<CUdevice> dev;                      // devices bound by this process
};

namespace {

bool multicast_supported(int device) {
  const Driver& d = drv();
  if (!d.ok) return false;
  CUdevice cd;
  int v = 0;
  if (d.DeviceGet(&cd, device) != CUDA_SUCCESS) return false;
  if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cd) != CUDA_SUCCESS) return false;
  return v != 0;
}

CUmemAccessDesc access_for(int device) {
  CUmemAccessDesc a;
  memset(&a, 0, sizeof(a));
  a.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  a.location.id = device;
  a.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  return a;
}

CUmemAllocationProp mem_prop(int device, bool shareable) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = shareable ? CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR : CU_MEM_HANDLE_TYPE_NONE;
  return p;
}

// mapped size for `bytes` on `n` GPUs: a multiple of the multicast and of the allocation granularity
bool region_size(int n, int device, bool shareable, bool with_mc, size_t bytes, size_t* size, size_t* gran) {
  const Driver& d = drv();
  size_t g = 0;
  CUmemAllocationProp p = mem_prop(device, shareable);
  if (d.MemGetAllocationGranularity(&g, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || g == 0) return false;
  if (with_mc) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = (unsigned)n;
    mp.size = round_up(bytes, g);
    mp.handleTypes = shareable ? CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR : 0;
    size_t mg = 0;
    if (d.MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || mg == 0) return false;
    if (mg > g) g = mg;
  }
  *gran = g;
  *size = round_up(bytes ? bytes : 1, g);
  return true;
}

// ---- file descriptors over a unix-domain socket ---------------------------------------------------
bool send_fd(int sock, int fd, int tag) {
  struct msghdr msg;
  memset(&msg, 0, sizeof(msg));
  struct iovec io = {&tag, sizeof(tag)};
  char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msg.msg_iov = &io;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  return sendmsg(sock, &msg, 0) == (ssize_t)sizeof(tag);
}
bool recv_fd(int sock, int* fd, int* tag) {
  struct msghdr msg;
  memset(&msg, 0, sizeof(msg));
  struct iovec io = {tag, sizeof(*tag)};
  char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msg.msg_iov = &io;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  if (recvmsg(sock, &msg, MSG_WAITALL) != (ssize_t)sizeof(*tag)) return false;
  struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
  if (!c || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) return false;
  memcpy(fd, CMSG_DATA(c), sizeof(int));
  return true;
}
bool send_int(int sock, int v) { return send(sock, &v, sizeof(v), 0) == (ssize_t)sizeof(v); }
bool recv_int(int sock, int* v) { return recv(sock, v, sizeof(*v), MSG_WAITALL) == (ssize_t)sizeof(*v); }

void set_timeouts(int sock, int seconds) {
  struct timeval tv = {seconds, 0};
  setsockopt(sock, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  setsockopt(sock, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
}

// abstract socket name (no file is left behind)
socklen_t abstract_addr(struct sockaddr_un* a, const char* session) {
  memset(a, 0, sizeof(*a));
  a->sun_family = AF_UNIX;
  const int len = snprintf(a->sun_path + 1, sizeof(a->sun_path) - 2, "hc_mc_%s", session);
  return (socklen_t)(offsetof(struct sockaddr_un, sun_path) + 1 + (len > 0 ? len : 0));
}

// Hub (rank 0) and spokes.  `socks`: on the hub the connection of every other rank (index = rank),
// on a spoke socks[0] is the connection to the hub.
bool hub_barrier(int rank, int world, std::vector<int>& socks) {
  int v = 0;
  if (rank == 0) {
    for (int r = 1; r < world; ++r)
      if (!recv_int(socks[r], &v)) return false;
    for (int r = 1; r < world; ++r)
      if (!send_int(socks[r], 1)) return false;
    return true;
  }
  return send_int(socks[0], 1) && recv_int(socks[0], &v);
}

void close_all(std::vector<int>& v) {
  for (int& s : v)
    if (s >= 0) {
      close(s);
      s = -1;
    }
}

}  // namespace

extern "C" {

int hc_multicast_supported(int device) { return multicast_supported(device) ? 1 : 0; }

void hc_mc_destroy(hc_mc_region* r) {
  if (!r) return;
  const Driver& d = drv();
  cudaDeviceSynchronize();
  if (r->mc_va) {
    d.MemUnmap(r->mc_va, r->size);
    d.MemAddressFree(r->mc_va, r->size);
  }
  if (r->has_mc)
    for (CUdevice cd : r->dev) d.MulticastUnbind(r->mc, cd, 0, r->size);
  for (size_t i = 0; i < r->uc.size(); ++i)
    if (r->uc[i]) {
      d.MemUnmap(r->uc[i], r->size);
      d.MemAddressFree(r->uc[i], r->size);
    }
  for (CUmemGenericAllocationHandle h : r->mem)
    if (h) d.MemRelease(h);
  if (r->has_mc) d.MemRelease(r->mc);
  delete r;
}

void* hc_mc_unicast_ptr(hc_mc_region* r, int idx) {
  return (r && idx >= 0 && idx < r->n) ? reinterpret_cast<void*>(r->uc[(size_t)idx]) : nullptr;
}
void* hc_mc_multicast_ptr(hc_mc_region* r) { return (r && r->has_mc) ? reinterpret_cast<void*>(r->mc_va) : nullptr; }
size_t hc_mc_bytes(hc_mc_region* r) { return r ? r->size : 0; }

// One process, n_dev GPUs.  Every region is zeroed.  Without multicast support on every GPU the
// regions are still created and mapped everywhere; hc_mc_multicast_ptr then returns NULL.
int hc_mc_create_local(hc_mc_region** out, int n_dev, const int* devices, size_t bytes) {
  const Driver& d = drv();
  if (!out || n_dev < 1 || n_dev > 8 || !devices || !d.ok) return hc::kErrArgument;
  int before = 0;
  cudaGetDevice(&before);
  bool with_mc = n_dev > 1;
  for (int i = 0; i < n_dev; ++i) {
    if (cudaSetDevice(devices[i]) != cudaSuccess || cudaFree(nullptr) != cudaSuccess) return hc::kErrCuda;
    with_mc = with_mc && multicast_supported(devices[i]);
  }
  hc_mc_region* r = new (std::nothrow) hc_mc_region();
  if (!r) return hc::kErrArgument;
  r->n = n_dev;
  r->mem.assign((size_t)n_dev, 0);
  r->uc.assign((size_t)n_dev, 0);
  size_t gran = 0;
  bool good = region_size(n_dev, devices[0], false, with_mc, bytes, &r->size, &gran);
  if (good && with_mc) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = (unsigned)n_dev;
    mp.size = r->size;
    good = d.MulticastCreate(&r->mc, &mp) == CUDA_SUCCESS;
    r->has_mc = good;
    for (int i = 0; good && i < n_dev; ++i) {
      CUdevice cd;
      good = d.DeviceGet(&cd, devices[i]) == CUDA_SUCCESS && d.MulticastAddDevice(r->mc, cd) == CUDA_SUCCESS;
      if (good) r->dev.push_back(cd);
    }
  }
  std::vector<CUmemAccessDesc> acc;
  for (int i = 0; i < n_dev; ++i) acc.push_back(access_for(devices[i]));
  for (int i = 0; good && i < n_dev; ++i) {
    CUmemAllocationProp p = mem_prop(devices[i], false);
    good = d.MemCreate(&r->mem[(size_t)i], r->size, &p, 0) == CUDA_SUCCESS &&
           d.MemAddressReserve(&r->uc[(size_t)i], r->size, gran, 0, 0) == CUDA_SUCCESS &&
           d.MemMap(r->uc[(size_t)i], r->size, 0, r->mem[(size_t)i], 0) == CUDA_SUCCESS &&
           d.MemSetAccess(r->uc[(size_t)i], r->size, acc.data(), acc.size()) == CUDA_SUCCESS;
    if (good && r->has_mc) good = d.MulticastBindMem(r->mc, 0, r->mem[(size_t)i], 0, r->size, 0) == CUDA_SUCCESS;
    if (good) good = cudaSetDevice(devices[i]) == cudaSuccess &&
                     cudaMemset(reinterpret_cast<void*>(r->uc[(size_t)i]), 0, r->size) == cudaSuccess &&
                     cudaDeviceSynchronize() == cudaSuccess;
  }
  if (good && r->has_mc)
    good = d.MemAddressReserve(&r->mc_va, r->size, gran, 0, 0) == CUDA_SUCCESS &&
           d.MemMap(r->mc_va, r->size, 0, r->mc, 0) == CUDA_SUCCESS &&
           d.MemSetAccess(r->mc_va, r->size, acc.data(), acc.size()) == CUDA_SUCCESS;
  cudaSetDevice(before);
  if (!good) {
    hc_mc_destroy(r);
    return hc::kErrCuda;
  }
  *out = r;
  return hc::kOk;
}

// One process per GPU (the current device of the caller).  Collective over the `world` ranks that
// pass the same `session` string (unique per communicator, e.g. "<port>_<counter>"); rank 0 is the
// hub of a unix-domain socket over which the handles travel as file descriptors.  Every region is
// zeroed before the call returns anywhere.  Falls back to peer mappings without a multicast alias
// where a GPU lacks multicast support (every rank must see the same answer).
int hc_mc_create_shared(hc_mc_region** out, int rank, int world, size_t bytes, const char* session) {
  const Driver& d = drv();
  if (!out || world < 1 || world > 8 || rank < 0 || rank >= world || !session || !d.ok) return hc::kErrArgument;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || cudaFree(nullptr) != cudaSuccess) return hc::kErrCuda;
  hc_mc_region* r = new (std::nothrow) hc_mc_region();
  if (!r) return hc::kErrArgument;
  r->n = world;
  r->own = rank;
  r->mem.assign((size_t)world, 0);
  r->uc.assign((size_t)world, 0);
  std::vector<int> socks((size_t)world, -1), fds((size_t)world, -1);
  int listener = -1, mc_fd = -1;
  int want_mc = (world > 1 && multicast_supported(device)) ? 1 : 0;
  size_t gran = 0;
  bool good = true;
  auto fail = [&](const char* what) {
    if (good) fprintf(stderr, "homcomp multicast bootstrap (rank %d): %s failed (errno %d)\n", rank, what, errno);
    good = false;
  };

  // ---- rendezvous -----------------------------------------------------------------------------------
  struct sockaddr_un addr;
  const socklen_t alen = abstract_addr(&addr, session);
  if (world > 1) {
    if (rank == 0) {
      listener = socket(AF_UNIX, SOCK_STREAM, 0);
      if (listener < 0 || bind(listener, (struct sockaddr*)&addr, alen) != 0 || listen(listener, world) != 0) fail("listen");
      if (good) set_timeouts(listener, 60);
      for (int k = 1; good && k < world; ++k) {
        int s = accept(listener, nullptr, nullptr);
        int who = -1;
        if (s < 0) { fail("accept"); break; }
        set_timeouts(s, 60);
        if (!recv_int(s, &who) || who < 1 || who >= world || socks[(size_t)who] >= 0) { close(s); fail("hello"); break; }
        socks[(size_t)who] = s;
      }
    } else {
      int s = socket(AF_UNIX, SOCK_STREAM, 0);
      if (s < 0) fail("socket");
      bool connected = false;
      for (int tries = 0; good && tries < 3000 && !connected; ++tries) {  // the hub may not be listening yet
        connected = connect(s, (struct sockaddr*)&addr, alen) == 0;
        if (!connected) usleep(10000);
      }
      if (good && !connected) fail("connect");
      if (good) {
        set_timeouts(s, 60);
        socks[0] = s;
        if (!send_int(s, rank)) fail("hello");
      } else if (s >= 0) {
        close(s);
      }
    }
    // multicast only if every GPU supports it: spokes report, the hub decides and tells
    if (good) {
      if (rank == 0) {
        for (int q = 1; q < world; ++q) {
          int v = 0;
          if (!recv_int(socks[(size_t)q], &v)) { fail("capability"); break; }
          want_mc = want_mc && v;
        }
        for (int q = 1; good && q < world; ++q)
          if (!send_int(socks[(size_t)q], want_mc)) fail("capability");
      } else if (!send_int(socks[0], want_mc) || !recv_int(socks[0], &want_mc)) {
        fail("capability");
      }
    }
  }

  // ---- this rank's memory, and on the hub the multicast object ----------------------------------------
  if (good && !region_size(world, device, world > 1, want_mc != 0, bytes, &r->size, &gran)) fail("granularity");
  if (good) {
    CUmemAllocationProp p = mem_prop(device, world > 1);
    if (d.MemCreate(&r->mem[(size_t)rank], r->size, &p, 0) != CUDA_SUCCESS) fail("cuMemCreate");
  }
  if (good && world > 1 &&
      d.MemExportToShareableHandle(&fds[(size_t)rank], r->mem[(size_t)rank], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) !=
          CUDA_SUCCESS)
    fail("export of the memory handle");
  if (good && want_mc && rank == 0) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = (unsigned)world;
    mp.size = r->size;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    if (d.MulticastCreate(&r->mc, &mp) != CUDA_SUCCESS) fail("cuMulticastCreate");
    else r->has_mc = true;
    if (good && d.MemExportToShareableHandle(&mc_fd, r->mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS)
      fail("export of the multicast handle");
  }

  // ---- handles: spokes -> hub, hub -> everybody -----------------------------------------------------------
  if (good && world > 1) {
    if (rank == 0) {
      for (int q = 1; good && q < world; ++q) {
        int tag = -1;
        if (!recv_fd(socks[(size_t)q], &fds[(size_t)q], &tag) || tag != q) fail("receiving a memory handle");
      }
      for (int q = 1; good && q < world; ++q) {
        for (int m = 0; good && m < world; ++m)
          if (m != q && !send_fd(socks[(size_t)q], fds[(size_t)m], m)) fail("sending a memory handle");
        if (good && want_mc && !send_fd(socks[(size_t)q], mc_fd, world)) fail("sending the multicast handle");
      }
    } else {
      if (!send_fd(socks[0], fds[(size_t)rank], rank)) fail("sending the memory handle");
      for (int k = 0; good && k < world - 1; ++k) {
        int fd = -1, tag = -1;
        if (!recv_fd(socks[0], &fd, &tag) || tag < 0 || tag >= world || tag == rank) { fail("receiving a memory handle"); break; }
        fds[(size_t)tag] = fd;
      }
      if (good && want_mc) {
        int tag = -1;
        if (!recv_fd(socks[0], &mc_fd, &tag) || tag != world) fail("receiving the multicast handle");
      }
    }
  }
  // ---- import, bind, map ----------------------------------------------------------------------------------
  for (int q = 0; good && q < world; ++q)
    if (q != rank && d.MemImportFromShareableHandle(&r->mem[(size_t)q], (void*)(uintptr_t)fds[(size_t)q],
                                                    CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS)
      fail("import of a memory handle");
  if (good && want_mc && rank != 0) {
    if (d.MemImportFromShareableHandle(&r->mc, (void*)(uintptr_t)mc_fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS)
      fail("import of the multicast handle");
    else r->has_mc = true;
  }
  CUdevice cd = 0;
  if (good && d.DeviceGet(&cd, device) != CUDA_SUCCESS) fail("cuDeviceGet");
  if (good && want_mc) {
    if (d.MulticastAddDevice(r->mc, cd) != CUDA_SUCCESS) fail("cuMulticastAddDevice");
    else r->dev.push_back(cd);
  }
  // every device has been added before anybody binds memory
  if (world > 1 && !hub_barrier(rank, world, socks)) fail("barrier after add-device");
  if (good && want_mc && d.MulticastBindMem(r->mc, 0, r->mem[(size_t)rank], 0, r->size, 0) != CUDA_SUCCESS) fail("cuMulticastBindMem");
  const CUmemAccessDesc acc = access_for(device);
  for (int q = 0; good && q < world; ++q)
    if (d.MemAddressReserve(&r->uc[(size_t)q], r->size, gran, 0, 0) != CUDA_SUCCESS ||
        d.MemMap(r->uc[(size_t)q], r->size, 0, r->mem[(size_t)q], 0) != CUDA_SUCCESS ||
        d.MemSetAccess(r->uc[(size_t)q], r->size, &acc, 1) != CUDA_SUCCESS)
      fail("mapping a region");
  if (good && want_mc &&
      (d.MemAddressReserve(&r->mc_va, r->size, gran, 0, 0) != CUDA_SUCCESS || d.MemMap(r->mc_va, r->size, 0, r->mc, 0) != CUDA_SUCCESS ||
       d.MemSetAccess(r->mc_va, r->size, &acc, 1) != CUDA_SUCCESS))
    fail("mapping the multicast object");
  if (good && (cudaMemset(reinterpret_cast<void*>(r->uc[(size_t)rank]), 0, r->size) != cudaSuccess ||
               cudaDeviceSynchronize() != cudaSuccess))
    fail("zeroing the region");
  // everybody's region is zeroed, bound and mapped before anybody's first store; the hub also learns
  // here whether a spoke failed on the way
  int all_good = good ? 1 : 0;
  if (world > 1) {
    if (rank == 0) {
      for (int q = 1; q < world; ++q) {
        int v = 0;
        if (socks[(size_t)q] < 0 || !recv_int(socks[(size_t)q], &v) || !v) all_good = 0;
      }
      for (int q = 1; q < world; ++q)
        if (socks[(size_t)q] >= 0) send_int(socks[(size_t)q], all_good);
    } else if (socks[0] < 0 || !send_int(socks[0], all_good) || !recv_int(socks[0], &all_good)) {
      all_good = 0;
    }
  }
  close_all(socks);
  if (listener >= 0) close(listener);
  for (int& fd : fds)
    if (fd >= 0) close(fd);  // the imported handles keep the memory alive
  if (mc_fd >= 0) close(mc_fd);
  if (!all_good) {
    hc_mc_destroy(r);
    return hc::kErrCuda;
  }
  *out = r;
  return hc::kOk;
}

}  // extern "C"
