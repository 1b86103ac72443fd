// NVLink multicast region (see mcast_region.h).  All driver entry points are looked up at run
// time (cudaGetDriverEntryPoint), so the library loads on machines without a driver.
#include "mcast_region.h"

#include <cuda.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <stdexcept>

namespace b200 {

namespace {

template <typename Fn>
Fn driver_fn(const char* name) {
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &ptr, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess ||
      ptr == nullptr) {
    throw std::runtime_error(std::string("driver entry point not available: ") + name);
  }
  return reinterpret_cast<Fn>(ptr);
}

void drv(CUresult r, const char* what) {
  if (r != CUDA_SUCCESS) throw std::runtime_error(std::string(what) + " failed with CUresult " + std::to_string((int)r));
}

struct Driver {
  CUresult (*DeviceGet)(CUdevice*, int);
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t,
                               unsigned long long);
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
};

const Driver& driver() {
  static const Driver d = [] {
    Driver x;
    x.DeviceGet = driver_fn<decltype(x.DeviceGet)>("cuDeviceGet");
    x.DeviceGetAttribute = driver_fn<decltype(x.DeviceGetAttribute)>("cuDeviceGetAttribute");
    x.MemCreate = driver_fn<decltype(x.MemCreate)>("cuMemCreate");
    x.MemRelease = driver_fn<decltype(x.MemRelease)>("cuMemRelease");
    x.MemAddressReserve = driver_fn<decltype(x.MemAddressReserve)>("cuMemAddressReserve");
    x.MemAddressFree = driver_fn<decltype(x.MemAddressFree)>("cuMemAddressFree");
    x.MemMap = driver_fn<decltype(x.MemMap)>("cuMemMap");
    x.MemUnmap = driver_fn<decltype(x.MemUnmap)>("cuMemUnmap");
    x.MemSetAccess = driver_fn<decltype(x.MemSetAccess)>("cuMemSetAccess");
    x.MemExportToShareableHandle = driver_fn<decltype(x.MemExportToShareableHandle)>("cuMemExportToShareableHandle");
    x.MemImportFromShareableHandle = driver_fn<decltype(x.MemImportFromShareableHandle)>("cuMemImportFromShareableHandle");
    x.MulticastCreate = driver_fn<decltype(x.MulticastCreate)>("cuMulticastCreate");
    x.MulticastAddDevice = driver_fn<decltype(x.MulticastAddDevice)>("cuMulticastAddDevice");
    x.MulticastBindMem = driver_fn<decltype(x.MulticastBindMem)>("cuMulticastBindMem");
    x.MulticastUnbind = driver_fn<decltype(x.MulticastUnbind)>("cuMulticastUnbind");
    x.MulticastGetGranularity = driver_fn<decltype(x.MulticastGetGranularity)>("cuMulticastGetGranularity");
    return x;
  }();
  return d;
}

struct DeviceScope {
  int prev = -1;
  explicit DeviceScope(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
    else prev = -1;
    cudaFree(nullptr);  // make sure the primary context exists before driver calls
  }
  ~DeviceScope() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

CUmulticastObjectProp mc_prop(int world, uint64_t bytes) {
  CUmulticastObjectProp prop = {};
  prop.numDevices = (unsigned)world;
  prop.size = bytes;
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  prop.flags = 0;
  return prop;
}

}  // namespace

bool McastRegion::supported(int device, std::string* why) {
  try {
    DeviceScope scope(device);
    const Driver& d = driver();
    CUdevice dev;
    drv(d.DeviceGet(&dev, device), "cuDeviceGet");
    int ok = 0;
    drv(d.DeviceGetAttribute(&ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev), "cuDeviceGetAttribute(MULTICAST_SUPPORTED)");
    if (!ok && why) *why = "CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED is 0";
    return ok != 0;
  } catch (const std::exception& e) {
    if (why) *why = e.what();
    return false;
  }
}

McastRegion::McastRegion(int rank, int world_size, uint64_t bytes, int device)
    : rank_(rank), world_(world_size), device_(device), bytes_(0), mc_handle_(0), mem_handle_(0), have_mc_(false),
      have_mem_(false), bound_(false), device_added_(false), local_va_(nullptr), mc_va_(nullptr), export_fd_(-1) {
  if (world_size < 2) throw std::runtime_error("a multicast region needs at least two ranks");
  DeviceScope scope(device_);
  const Driver& d = driver();
  CUmulticastObjectProp prop = mc_prop(world_, bytes);
  size_t gran = 0;
  drv(d.MulticastGetGranularity(&gran, &prop, CU_MULTICAST_GRANULARITY_RECOMMENDED), "cuMulticastGetGranularity");
  if (gran == 0) gran = 2u << 20;
  bytes_ = (bytes + gran - 1) / gran * gran;
}

McastRegion::~McastRegion() {
  try {
    close();
  } catch (...) {
  }
}

int McastRegion::create_and_export() {
  DeviceScope scope(device_);
  const Driver& d = driver();
  CUmulticastObjectProp prop = mc_prop(world_, bytes_);
  CUmemGenericAllocationHandle h;
  drv(d.MulticastCreate(&h, &prop), "cuMulticastCreate");
  mc_handle_ = h;
  have_mc_ = true;
  int fd = -1;
  drv(d.MemExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
  export_fd_ = fd;
  return fd;
}

void McastRegion::import_from(int64_t pid, int fd) {
  // duplicate the exporting process's descriptor into this process
  const long pidfd = syscall(SYS_pidfd_open, (pid_t)pid, 0);
  if (pidfd < 0) throw std::runtime_error("pidfd_open failed (cannot reach the exporting process)");
  const long mine = syscall(SYS_pidfd_getfd, (int)pidfd, fd, 0);
  ::close((int)pidfd);
  if (mine < 0) throw std::runtime_error("pidfd_getfd failed (no permission to duplicate the peer's descriptor)");
  DeviceScope scope(device_);
  const Driver& d = driver();
  CUmemGenericAllocationHandle h;
  const CUresult r = d.MemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(mine)),
                                                    CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  ::close((int)mine);
  drv(r, "cuMemImportFromShareableHandle");
  mc_handle_ = h;
  have_mc_ = true;
}

void McastRegion::add_device() {
  if (!have_mc_) throw std::runtime_error("add_device: no multicast object yet");
  DeviceScope scope(device_);
  const Driver& d = driver();
  CUdevice dev;
  drv(d.DeviceGet(&dev, device_), "cuDeviceGet");
  drv(d.MulticastAddDevice(mc_handle_, dev), "cuMulticastAddDevice");
  device_added_ = true;
}

void McastRegion::bind_and_map() {
  if (!device_added_) throw std::runtime_error("bind_and_map: add_device first");
  DeviceScope scope(device_);
  const Driver& d = driver();
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device_;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle mem;
  drv(d.MemCreate(&mem, bytes_, &prop, 0), "cuMemCreate");
  mem_handle_ = mem;
  have_mem_ = true;
  CUmemAccessDesc access = {};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device_;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CUdeviceptr va = 0;
  drv(d.MemAddressReserve(&va, bytes_, bytes_ >= (2u << 20) ? (2u << 20) : 0, 0, 0), "cuMemAddressReserve(local)");
  local_va_ = reinterpret_cast<void*>(va);
  drv(d.MemMap(va, bytes_, 0, mem, 0), "cuMemMap(local)");
  drv(d.MemSetAccess(va, bytes_, &access, 1), "cuMemSetAccess(local)");
  if (cudaMemset(local_va_, 0, bytes_) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess)
    throw std::runtime_error("cudaMemset of the multicast-bound memory failed");
  drv(d.MulticastBindMem(mc_handle_, 0, mem, 0, bytes_, 0), "cuMulticastBindMem");
  bound_ = true;
  CUdeviceptr mva = 0;
  drv(d.MemAddressReserve(&mva, bytes_, bytes_ >= (2u << 20) ? (2u << 20) : 0, 0, 0), "cuMemAddressReserve(multicast)");
  mc_va_ = reinterpret_cast<void*>(mva);
  drv(d.MemMap(mva, bytes_, 0, mc_handle_, 0), "cuMemMap(multicast)");
  drv(d.MemSetAccess(mva, bytes_, &access, 1), "cuMemSetAccess(multicast)");
}

void McastRegion::close() {
  if (!have_mc_ && !have_mem_ && local_va_ == nullptr && mc_va_ == nullptr) return;
  DeviceScope scope(device_);
  const Driver& d = driver();
  cudaDeviceSynchronize();
  if (mc_va_ != nullptr) {
    d.MemUnmap(reinterpret_cast<CUdeviceptr>(mc_va_), bytes_);
    d.MemAddressFree(reinterpret_cast<CUdeviceptr>(mc_va_), bytes_);
    mc_va_ = nullptr;
  }
  if (bound_) {
    CUdevice dev;
    if (d.DeviceGet(&dev, device_) == CUDA_SUCCESS) d.MulticastUnbind(mc_handle_, dev, 0, bytes_);
    bound_ = false;
  }
  if (local_va_ != nullptr) {
    d.MemUnmap(reinterpret_cast<CUdeviceptr>(local_va_), bytes_);
    d.MemAddressFree(reinterpret_cast<CUdeviceptr>(local_va_), bytes_);
    local_va_ = nullptr;
  }
  if (have_mem_) {
    d.MemRelease(mem_handle_);
    have_mem_ = false;
  }
  if (have_mc_) {
    d.MemRelease(mc_handle_);
    have_mc_ = false;
  }
  if (export_fd_ >= 0) {
    ::close(export_fd_);
    export_fd_ = -1;
  }
}

// ---------------------------------------------------------------------------------------
__global__ void mcast_selftest_kernel(const uint8_t* mc, uint4* out, uint64_t n_vec) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (uint64_t)gridDim.x * blockDim.x) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc + i * 16)
                 : "memory");
    out[i] = v;
  }
}

cudaError_t launch_mcast_selftest(const McastRegion& region, uint64_t offset, void* out, uint64_t n_vec,
                                  cudaStream_t stream) {
  if (!region.mapped() || (offset & 15) || offset + n_vec * 16 > region.bytes()) return cudaErrorInvalidValue;
  const int grid = (int)((n_vec + 255) / 256 < 148 ? (n_vec + 255) / 256 : 148);
  mcast_selftest_kernel<<<grid < 1 ? 1 : grid, 256, 0, stream>>>(static_cast<const uint8_t*>(region.mc_ptr()) + offset,
                                                                static_cast<uint4*>(out), n_vec);
  return cudaGetLastError();
}

}  // namespace b200
