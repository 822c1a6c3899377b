// One contiguous virtual address range whose sections are backed by device memory or by pinned host memory
// (dist_moe/_vmm.py:149-427 `VMMRegion`).  The activation arena of a context with `Config.vmm` is such a range:
// [device: activation slots | host: overflow scratch | device: hot scratch].  The device planner carves scratch from
// the top of the range downwards, so a balanced step never leaves device memory and only a step whose routing
// overflows the hot section touches the host section (over PCIe / the chip-to-chip link).
//
// Driver calls are fetched through cudaGetDriverEntryPoint, so the library has no link-time dependency on libcuda.
#include <cuda.h>

#include <cstdint>
#include <vector>

#include "common.cuh"
#include "../../include/dist_moe_b200.h"

namespace dm {

struct DriverVmm {
  CUresult (*get_granularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*address_reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*address_free)(CUdeviceptr, size_t);
  CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*release)(CUmemGenericAllocationHandle);
  CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*unmap)(CUdeviceptr, size_t);
  CUresult (*set_access)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*device_get_attribute)(int*, CUdevice_attribute, CUdevice);
  bool ok;
};

template <class Fn>
static bool load_entry(const char* name, Fn* out) {
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &sym, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess ||
      sym == nullptr)
    return false;
  *out = reinterpret_cast<Fn>(sym);
  return true;
}

static const DriverVmm& driver() {
  static DriverVmm d = [] {
    DriverVmm v{};
    v.ok = load_entry("cuMemGetAllocationGranularity", &v.get_granularity) &&
           load_entry("cuMemAddressReserve", &v.address_reserve) && load_entry("cuMemAddressFree", &v.address_free) &&
           load_entry("cuMemCreate", &v.create) && load_entry("cuMemRelease", &v.release) &&
           load_entry("cuMemMap", &v.map) && load_entry("cuMemUnmap", &v.unmap) &&
           load_entry("cuMemSetAccess", &v.set_access) && load_entry("cuDeviceGetAttribute", &v.device_get_attribute);
    return v;
  }();
  return d;
}

static CUmemAllocationProp device_prop(int device) {
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  return prop;
}

struct VmmRegion {
  int device = 0;
  CUdeviceptr base = 0;
  size_t total = 0;
  std::vector<size_t> offsets, sizes;
  std::vector<CUmemGenericAllocationHandle> handles;
  std::vector<char> mapped;
};

// Unmaps, releases and frees whatever the region still owns; keeps going after a failure and reports the first one.
static int region_release(VmmRegion* r) {
  const DriverVmm& d = driver();
  int first = 0;
  for (size_t i = r->handles.size(); i-- > 0;) {
    if (r->mapped[i]) {
      const CUresult e = d.unmap(r->base + r->offsets[i], r->sizes[i]);
      if (e == CUDA_SUCCESS)
        r->mapped[i] = 0;
      else if (!first)
        first = 1000 + static_cast<int>(e);
    }
    if (!r->mapped[i] && r->handles[i] != 0) {
      const CUresult e = d.release(r->handles[i]);
      if (e == CUDA_SUCCESS)
        r->handles[i] = 0;
      else if (!first)
        first = 1000 + static_cast<int>(e);
    }
  }
  if (!first && r->base != 0) {
    const CUresult e = d.address_free(r->base, r->total);
    if (e == CUDA_SUCCESS)
      r->base = 0;
    else
      first = 1000 + static_cast<int>(e);
  }
  return first;
}

}  // namespace dm

using namespace dm;

extern "C" int dm_vmm_granularity(int device, int64_t* granularity_bytes) {
  if (!granularity_bytes || device < 0) return kRcBadArg;
  const DriverVmm& d = driver();
  if (!d.ok) return kRcNoDriver;
  const CUmemAllocationProp prop = device_prop(device);
  size_t g = 0;
  const CUresult e = d.get_granularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (e != CUDA_SUCCESS) return 1000 + static_cast<int>(e);
  *granularity_bytes = static_cast<int64_t>(g);
  return kRcOk;
}

extern "C" int dm_vmm_create(int device, int num_sections, const int64_t* section_bytes, const int* section_is_host,
                             uint64_t* base_out, void** region_out) {
  if (!section_bytes || !section_is_host || !base_out || !region_out || num_sections <= 0 || device < 0)
    return kRcBadArg;
  const DriverVmm& d = driver();
  if (!d.ok) return kRcNoDriver;
  int64_t granularity = 0;
  int rc = dm_vmm_granularity(device, &granularity);
  if (rc != kRcOk) return rc;
  VmmRegion* r = new VmmRegion();
  r->device = device;
  for (int i = 0; i < num_sections; ++i) {
    if (section_bytes[i] <= 0 || (section_bytes[i] % granularity) != 0) {
      delete r;
      return kRcBadArg;  // sections are sized by the plan, already rounded to the granularity
    }
    r->offsets.push_back(r->total);
    r->sizes.push_back(static_cast<size_t>(section_bytes[i]));
    r->total += static_cast<size_t>(section_bytes[i]);
  }
  r->handles.assign(num_sections, 0);
  r->mapped.assign(num_sections, 0);
  CUresult e = d.address_reserve(&r->base, r->total, static_cast<size_t>(granularity), 0, 0);
  if (e != CUDA_SUCCESS) {
    delete r;
    return 1000 + static_cast<int>(e);
  }
  // Host sections sit on the NUMA node next to the GPU where the driver names one, else on generic host memory.
  CUmemAllocationProp host_prop{};
  host_prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  int numa = -1;
  if (d.device_get_attribute(&numa, CU_DEVICE_ATTRIBUTE_HOST_NUMA_ID, device) == CUDA_SUCCESS && numa >= 0) {
    host_prop.location.type = CU_MEM_LOCATION_TYPE_HOST_NUMA;
    host_prop.location.id = numa;
  } else {
    host_prop.location.type = CU_MEM_LOCATION_TYPE_HOST;
    host_prop.location.id = 0;
  }
  const CUmemAllocationProp dev_prop = device_prop(device);
  for (int i = 0; i < num_sections && e == CUDA_SUCCESS; ++i) {
    e = d.create(&r->handles[i], r->sizes[i], section_is_host[i] ? &host_prop : &dev_prop, 0);
    if (e != CUDA_SUCCESS && section_is_host[i] && host_prop.location.type == CU_MEM_LOCATION_TYPE_HOST_NUMA) {
      CUmemAllocationProp plain = host_prop;  // a node the process may not allocate on: fall back to generic host
      plain.location.type = CU_MEM_LOCATION_TYPE_HOST;
      plain.location.id = 0;
      e = d.create(&r->handles[i], r->sizes[i], &plain, 0);
    }
    if (e != CUDA_SUCCESS) r->handles[i] = 0;
  }
  for (int i = 0; i < num_sections && e == CUDA_SUCCESS; ++i) {
    e = d.map(r->base + r->offsets[i], r->sizes[i], 0, r->handles[i], 0);
    if (e == CUDA_SUCCESS) r->mapped[i] = 1;
  }
  if (e == CUDA_SUCCESS) {
    CUmemAccessDesc access{};
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = device;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    e = d.set_access(r->base, r->total, &access, 1);
  }
  if (e != CUDA_SUCCESS) {
    region_release(r);
    delete r;
    return 1000 + static_cast<int>(e);
  }
  *base_out = static_cast<uint64_t>(r->base);
  *region_out = r;
  return kRcOk;
}

// Returns 0 and frees the handle when everything was released; after a failure the handle stays valid so that the
// call can be repeated (dist_moe/_vmm.py:372-427 keeps failed resources for a retry in the same way).
extern "C" int dm_vmm_destroy(void* region) {
  if (!region) return kRcBadArg;
  if (!driver().ok) return kRcNoDriver;
  VmmRegion* r = static_cast<VmmRegion*>(region);
  const int rc = region_release(r);
  if (rc == 0) delete r;
  return rc;
}
