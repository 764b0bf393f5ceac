// Virtual-memory backend of the symmetric heap, with NVLink multicast (NVLS).
//
// Slabs are created with cuMemCreate as shareable POSIX file descriptors.  Each
// rank runs a tiny descriptor server on an abstract Unix socket; a peer connects,
// asks for the slab (or, from heap rank 0, the multicast object) and receives the
// descriptor with SCM_RIGHTS, imports it and maps it.  When the device supports
// multicast, rank 0 creates one multicast object for the whole heap, every rank
// adds its device and binds its slab, and the object is mapped once more as
// `mc_base`: a store there lands in every slab, a multimem.ld_reduce there
// returns the sum over all slabs, both performed by the NVSwitch.
//
// Driver entry points are fetched with cudaGetDriverEntryPoint, so the library
// has no link-time dependency on libcuda and still loads on a machine without a
// GPU driver.
#include "cuda_state.h"
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>
#include <atomic>
#include <cstring>
#include <thread>

namespace tmpi {
namespace {

template <typename F> F drv(const char* name) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return reinterpret_cast<F>(fn);
}

#define DRV(name) static auto p_##name = drv<decltype(&name)>(#name); \
  if (!p_##name) return fail(TMPI_ERR_UNSUPPORTED, "driver entry point %s not found", #name)

#define CU(call)                                    \
  do {                                              \
    CUresult r__ = (call);                          \
    if (r__ != CUDA_SUCCESS) return cu_fail(r__, #call); \
  } while (0)

struct Blob { int pid; int rank; char sock[64]; };

int g_listen_fd = -1;
std::thread g_server;
std::atomic<bool> g_server_stop{false};

int send_fd(int sock, int fd) {
  char byte = 'F';
  iovec iov{&byte, 1};
  char ctrl[CMSG_SPACE(sizeof(int))] = {};
  msghdr msg{};
  msg.msg_iov = &iov; msg.msg_iovlen = 1; msg.msg_control = ctrl; msg.msg_controllen = sizeof(ctrl);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET; c->cmsg_type = SCM_RIGHTS; c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  return sendmsg(sock, &msg, 0) == 1 ? 0 : -1;
}

int recv_fd(int sock) {
  char byte = 0;
  iovec iov{&byte, 1};
  char ctrl[CMSG_SPACE(sizeof(int))] = {};
  msghdr msg{};
  msg.msg_iov = &iov; msg.msg_iovlen = 1; msg.msg_control = ctrl; msg.msg_controllen = sizeof(ctrl);
  if (recvmsg(sock, &msg, 0) != 1) return -1;
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  if (!c || c->cmsg_type != SCM_RIGHTS) return -1;
  int fd = -1;
  memcpy(&fd, CMSG_DATA(c), sizeof(int));
  return fd;
}

void make_addr(sockaddr_un* a, socklen_t* len, const char* name) {
  memset(a, 0, sizeof(*a));
  a->sun_family = AF_UNIX;
  size_t n = strlen(name);
  memcpy(a->sun_path + 1, name, n);            // abstract namespace: leading NUL
  *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

void serve(CudaHeap* h) {
  while (!g_server_stop.load()) {
    int c = accept(g_listen_fd, nullptr, nullptr);
    if (c < 0) break;
    char req = 0;
    if (read(c, &req, 1) == 1) {
      int fd = req == 'M' ? h->mc_export_fd : h->export_fd;
      if (fd >= 0) send_fd(c, fd);
    }
    close(c);
  }
}

int request_fd(const char* sock_name, char what) {
  int s = socket(AF_UNIX, SOCK_STREAM, 0);
  if (s < 0) return -1;
  sockaddr_un a; socklen_t len;
  make_addr(&a, &len, sock_name);
  int fd = -1;
  for (int attempt = 0; attempt < 200; ++attempt) {      // the peer may still be starting its server
    if (connect(s, (sockaddr*)&a, len) == 0) {
      if (write(s, &what, 1) == 1) fd = recv_fd(s);
      break;
    }
    usleep(10000);
  }
  close(s);
  return fd;
}

size_t g_gran = 0;

int map_handle(CudaHeap& h, CUmemGenericAllocationHandle handle, char** out) {
  DRV(cuMemAddressReserve); DRV(cuMemMap); DRV(cuMemSetAccess);
  CUdeviceptr va = 0;
  CU(p_cuMemAddressReserve(&va, h.total_bytes, g_gran, 0, 0));
  CU(p_cuMemMap(va, h.total_bytes, 0, handle, 0));
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE; acc.location.id = h.device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CU(p_cuMemSetAccess(va, h.total_bytes, &acc, 1));
  *out = (char*)va;
  return TMPI_OK;
}

}  // namespace

int cu_fail(CUresult r, const char* what) {
  static auto p_err = drv<decltype(&cuGetErrorString)>("cuGetErrorString");
  const char* s = nullptr;
  if (p_err) p_err(r, &s);
  return fail(TMPI_ERR_CUDA, "%s: %s (CUresult %d)", what, s ? s : "?", (int)r);
}

int vmm_create(CudaHeap& h) {
  DRV(cuMemGetAllocationGranularity); DRV(cuMemCreate); DRV(cuMemExportToShareableHandle);
  DRV(cuDeviceGetAttribute); DRV(cuMulticastGetGranularity);
  cudaFree(0);   // make sure the primary context exists
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE; prop.location.id = h.device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  CU(p_cuMemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  int mc_ok = 0;
  CU(p_cuDeviceGetAttribute(&mc_ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, h.device));
  if (mc_ok && h.world > 1 && tunable("use_nvls")) {
    CUmulticastObjectProp mp{};
    mp.numDevices = h.world; mp.size = h.total_bytes; mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (p_cuMulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran) gran = mg;
  }
  g_gran = gran;
  h.total_bytes = (h.total_bytes + gran - 1) / gran * gran;
  CU(p_cuMemCreate(&h.mem_handle, h.total_bytes, &prop, 0));
  int st = map_handle(h, h.mem_handle, &h.base[h.rank]);
  if (st) return st;
  CU(p_cuMemExportToShareableHandle(&h.export_fd, h.mem_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));

  // descriptor server
  g_listen_fd = socket(AF_UNIX, SOCK_STREAM, 0);
  if (g_listen_fd < 0) return fail(TMPI_ERR_SYS, "socket: %s", strerror(errno));
  char name[64];
  snprintf(name, sizeof(name), "tmpi_%d_%d", (int)getpid(), h.rank);
  sockaddr_un a; socklen_t len;
  make_addr(&a, &len, name);
  if (bind(g_listen_fd, (sockaddr*)&a, len) != 0 || listen(g_listen_fd, 64) != 0)
    return fail(TMPI_ERR_SYS, "bind/listen %s: %s", name, strerror(errno));
  g_server_stop.store(false);
  g_server = std::thread(serve, &h);
  return TMPI_OK;
}

int vmm_export(CudaHeap& h, void* out, int cap) {
  if (cap < (int)sizeof(Blob)) return -fail(TMPI_ERR_INVALID, "export buffer too small");
  Blob b{};
  b.pid = (int)getpid(); b.rank = h.rank;
  snprintf(b.sock, sizeof(b.sock), "tmpi_%d_%d", b.pid, h.rank);
  memcpy(out, &b, sizeof(b));
  return (int)sizeof(b);
}

int vmm_import(CudaHeap& h, int peer, const void* blob, int len) {
  DRV(cuMemImportFromShareableHandle);
  if (len != (int)sizeof(Blob)) return fail(TMPI_ERR_INVALID, "bad VMM blob length %d", len);
  Blob b;
  memcpy(&b, blob, sizeof(b));
  int fd = request_fd(b.sock, 'S');
  if (fd < 0) return fail(TMPI_ERR_SYS, "could not obtain the slab descriptor of rank %d", peer);
  CUresult r = p_cuMemImportFromShareableHandle(&h.peer_handles[peer], (void*)(uintptr_t)fd,
                                                CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  close(fd);
  if (r != CUDA_SUCCESS) return cu_fail(r, "cuMemImportFromShareableHandle");
  int st = map_handle(h, h.peer_handles[peer], &h.base[peer]);
  if (st) return st;
  h.imported[peer] = true;
  return TMPI_OK;
}

int vmm_destroy(CudaHeap& h) {
  DRV(cuMemUnmap); DRV(cuMemRelease); DRV(cuMemAddressFree); DRV(cuMulticastUnbind);
  if (h.mc_handle) {
    if (h.mc_bound) p_cuMulticastUnbind(h.mc_handle, h.device, 0, h.total_bytes);
    if (h.mc_base) { p_cuMemUnmap((CUdeviceptr)h.mc_base, h.total_bytes); p_cuMemAddressFree((CUdeviceptr)h.mc_base, h.total_bytes); }
    p_cuMemRelease(h.mc_handle);
    h.mc_handle = 0; h.mc_base = nullptr; h.mc_bound = false;
  }
  for (int r = 0; r < h.world; ++r) {
    if (!h.base[r]) continue;
    p_cuMemUnmap((CUdeviceptr)h.base[r], h.total_bytes);
    p_cuMemAddressFree((CUdeviceptr)h.base[r], h.total_bytes);
    if (r != h.rank && h.peer_handles[r]) { p_cuMemRelease(h.peer_handles[r]); h.peer_handles[r] = 0; }
  }
  if (h.mem_handle) { p_cuMemRelease(h.mem_handle); h.mem_handle = 0; }
  g_server_stop.store(true);
  if (g_listen_fd >= 0) { shutdown(g_listen_fd, SHUT_RDWR); close(g_listen_fd); g_listen_fd = -1; }
  if (g_server.joinable()) g_server.join();
  if (h.export_fd >= 0) { close(h.export_fd); h.export_fd = -1; }
  if (h.mc_export_fd >= 0) { close(h.mc_export_fd); h.mc_export_fd = -1; }
  return TMPI_OK;
}

}  // namespace tmpi

using namespace tmpi;

extern "C" {

// Heap rank 0 creates the multicast object and returns the blob to publish; other ranks get 0 bytes.
int tmpi_cuda_heap_mc_export(void* out, int cap) {
  CudaHeap& h = heap();
  if (!h.live || h.backend != 1 || h.world < 2) return 0;
  DRV(cuDeviceGetAttribute); DRV(cuMulticastCreate); DRV(cuMemExportToShareableHandle);
  int mc_ok = 0;
  if (p_cuDeviceGetAttribute(&mc_ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, h.device) != CUDA_SUCCESS || !mc_ok ||
      !tunable("use_nvls"))
    return 0;
  if (h.rank != 0) return 0;
  CUmulticastObjectProp mp{};
  mp.numDevices = h.world; mp.size = h.total_bytes; mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUresult r = p_cuMulticastCreate(&h.mc_handle, &mp);
  if (r != CUDA_SUCCESS) { cu_fail(r, "cuMulticastCreate"); h.mc_handle = 0; return 0; }
  r = p_cuMemExportToShareableHandle(&h.mc_export_fd, h.mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) { cu_fail(r, "export multicast"); return 0; }
  return vmm_export(h, out, cap);
}

// Every rank: import rank 0's object (rank 0 already holds it) and add this device.
int tmpi_cuda_heap_mc_import(const void* blob, int len) {
  CudaHeap& h = heap();
  if (!h.live || h.backend != 1) return fail(TMPI_ERR_STATE, "multicast needs the VMM backend");
  DRV(cuMemImportFromShareableHandle); DRV(cuMulticastAddDevice);
  if (h.rank != 0) {
    if (len != (int)sizeof(Blob)) return fail(TMPI_ERR_INVALID, "bad multicast blob");
    Blob b;
    memcpy(&b, blob, sizeof(b));
    int fd = request_fd(b.sock, 'M');
    if (fd < 0) return fail(TMPI_ERR_SYS, "could not obtain the multicast descriptor");
    CUresult r = p_cuMemImportFromShareableHandle(&h.mc_handle, (void*)(uintptr_t)fd,
                                                  CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    close(fd);
    if (r != CUDA_SUCCESS) { h.mc_handle = 0; return cu_fail(r, "import multicast"); }
  }
  CU(p_cuMulticastAddDevice(h.mc_handle, h.device));
  return TMPI_OK;
}

// After every rank has added its device: bind the slab and map the multicast view.
int tmpi_cuda_heap_mc_bind(void) {
  CudaHeap& h = heap();
  if (!h.live || !h.mc_handle) return fail(TMPI_ERR_STATE, "no multicast object");
  DRV(cuMulticastBindMem);
  CU(p_cuMulticastBindMem(h.mc_handle, 0, h.mem_handle, 0, h.total_bytes, 0));
  h.mc_bound = true;
  return map_handle(h, h.mc_handle, &h.mc_base);
}

}  // extern "C"
