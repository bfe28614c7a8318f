// Sleep-mode device allocator: every allocation is a reserved virtual range backed by a physical
// handle from the CUDA driver's virtual-memory API, so the physical memory can be released ("sleep")
// and re-created at the SAME address ("wake") without invalidating any pointer held by PyTorch,
// CUDA graphs or the engine.
//
// This file is a CPython extension module (`_b200_cumem`) that also exports the two C symbols
// `b200_cumem_malloc` / `b200_cumem_free` which torch.cuda.memory.CUDAPluggableAllocator calls.
// The allocation table lives here (ptr -> device, size, tag, mapped); Python drives policy:
//     set_tag(str)            tag given to allocations made from now on
//     allocations()           [(ptr, size, device, tag, mapped)]
//     release(ptr)            unmap + free the physical handle, keep the address range
//     restore(ptr)            create a new physical handle and map it at the same address
//     stats()                 {"mapped_bytes", "reserved_bytes", "allocations"}
//     use_fake_driver(bool)   host-memory emulation of the driver calls (CPU tests of the bookkeeping)
// The driver is loaded with dlopen at first use, so importing the module needs no GPU.
// Parity: csrc/cumem_allocator.cpp (777 lines) and vllm_metax/device_allocator/cumem.py:85-316
// of the reference (my_malloc / my_free, python_create_and_map, python_unmap_and_release).
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <cuda.h>
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>

namespace {

struct Driver {
  CUresult (*memCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*memRelease)(CUmemGenericAllocationHandle);
  CUresult (*memAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*memAddressFree)(CUdeviceptr, size_t);
  CUresult (*memMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*memUnmap)(CUdeviceptr, size_t);
  CUresult (*memSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*memGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*getErrorString)(CUresult, const char**);
  CUresult (*ctxGetCurrent)(CUcontext*);
  CUresult (*devicePrimaryCtxRetain)(CUcontext*, CUdevice);
  CUresult (*ctxSetCurrent)(CUcontext);
  CUresult (*memcpyDtoH)(void*, CUdeviceptr, size_t);
  CUresult (*memcpyHtoD)(CUdeviceptr, const void*, size_t);
  bool loaded = false;
};

Driver g_drv;
bool g_fake = false;
std::mutex g_mu;
std::string g_tag = "default";
std::string g_last_error;

struct Block {
  int device;
  size_t size;          // padded to the granularity
  size_t requested;
  std::string tag;
  CUmemGenericAllocationHandle handle;
  bool mapped;
};
std::map<unsigned long long, Block> g_blocks;

template <typename F>
bool sym(void* lib, const char* name, F& out) {
  out = reinterpret_cast<F>(dlsym(lib, name));
  return out != nullptr;
}

bool load_driver() {
  if (g_drv.loaded) return true;
  void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) lib = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) {
    g_last_error = "libcuda.so.1 not found";
    return false;
  }
  bool ok = sym(lib, "cuMemCreate", g_drv.memCreate) && sym(lib, "cuMemRelease", g_drv.memRelease) &&
            sym(lib, "cuMemAddressReserve", g_drv.memAddressReserve) &&
            sym(lib, "cuMemAddressFree", g_drv.memAddressFree) && sym(lib, "cuMemMap", g_drv.memMap) &&
            sym(lib, "cuMemUnmap", g_drv.memUnmap) && sym(lib, "cuMemSetAccess", g_drv.memSetAccess) &&
            sym(lib, "cuMemGetAllocationGranularity", g_drv.memGetAllocationGranularity) &&
            sym(lib, "cuGetErrorString", g_drv.getErrorString) && sym(lib, "cuCtxGetCurrent", g_drv.ctxGetCurrent) &&
            sym(lib, "cuDevicePrimaryCtxRetain", g_drv.devicePrimaryCtxRetain) &&
            sym(lib, "cuCtxSetCurrent", g_drv.ctxSetCurrent) && sym(lib, "cuMemcpyDtoH_v2", g_drv.memcpyDtoH) &&
            sym(lib, "cuMemcpyHtoD_v2", g_drv.memcpyHtoD);
  if (!ok) g_last_error = "CUDA driver lacks the virtual memory management entry points";
  g_drv.loaded = ok;
  return ok;
}

bool check(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return true;
  const char* msg = nullptr;
  if (g_drv.getErrorString) g_drv.getErrorString(r, &msg);
  g_last_error = std::string(what) + ": " + (msg ? msg : "unknown driver error") + " (" + std::to_string((int)r) + ")";
  return false;
}

CUmemAllocationProp props_for(int device) {
  CUmemAllocationProp p;
  std::memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  return p;
}

bool ensure_context(int device) {
  CUcontext ctx = nullptr;
  if (!check(g_drv.ctxGetCurrent(&ctx), "cuCtxGetCurrent")) return false;
  if (ctx) return true;
  if (!check(g_drv.devicePrimaryCtxRetain(&ctx, device), "cuDevicePrimaryCtxRetain")) return false;
  return check(g_drv.ctxSetCurrent(ctx), "cuCtxSetCurrent");
}

size_t granularity(int device) {
  if (g_fake) return 2u << 20;
  CUmemAllocationProp p = props_for(device);
  size_t g = 0;
  if (!check(g_drv.memGetAllocationGranularity(&g, &p, CU_MEM_ALLOC_GRANULARITY_MINIMUM), "granularity") || g == 0)
    g = 2u << 20;
  return g;
}

// physical handle + map + access at `addr`
bool back_range(unsigned long long addr, Block& b) {
  if (g_fake) {
    b.handle = 1;
    b.mapped = true;
    return true;
  }
  CUmemAllocationProp p = props_for(b.device);
  if (!check(g_drv.memCreate(&b.handle, b.size, &p, 0), "cuMemCreate")) return false;
  if (!check(g_drv.memMap((CUdeviceptr)addr, b.size, 0, b.handle, 0), "cuMemMap")) {
    g_drv.memRelease(b.handle);
    return false;
  }
  CUmemAccessDesc acc;
  std::memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = b.device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (!check(g_drv.memSetAccess((CUdeviceptr)addr, b.size, &acc, 1), "cuMemSetAccess")) {
    g_drv.memUnmap((CUdeviceptr)addr, b.size);
    g_drv.memRelease(b.handle);
    return false;
  }
  b.mapped = true;
  return true;
}

bool unback_range(unsigned long long addr, Block& b) {
  if (!b.mapped) return true;
  if (!g_fake) {
    if (!check(g_drv.memUnmap((CUdeviceptr)addr, b.size), "cuMemUnmap")) return false;
    if (!check(g_drv.memRelease(b.handle), "cuMemRelease")) return false;
  }
  b.mapped = false;
  b.handle = 0;
  return true;
}

unsigned long long do_alloc(size_t size, int device) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_fake && (!load_driver() || !ensure_context(device))) return 0;
  const size_t g = granularity(device);
  Block b{device, (size + g - 1) / g * g, size, g_tag, 0, false};
  unsigned long long addr = 0;
  if (g_fake) {
    addr = reinterpret_cast<unsigned long long>(std::malloc(b.size));
    if (!addr) return 0;
  } else {
    CUdeviceptr va = 0;
    if (!check(g_drv.memAddressReserve(&va, b.size, g, 0, 0), "cuMemAddressReserve")) return 0;
    addr = (unsigned long long)va;
  }
  if (!back_range(addr, b)) {
    if (g_fake) std::free(reinterpret_cast<void*>(addr));
    else g_drv.memAddressFree((CUdeviceptr)addr, b.size);
    return 0;
  }
  g_blocks[addr] = b;
  return addr;
}

bool do_free(unsigned long long addr) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_blocks.find(addr);
  if (it == g_blocks.end()) {
    g_last_error = "free of an address this allocator does not own";
    return false;
  }
  bool ok = unback_range(addr, it->second);
  if (g_fake) std::free(reinterpret_cast<void*>(addr));
  else ok = check(g_drv.memAddressFree((CUdeviceptr)addr, it->second.size), "cuMemAddressFree") && ok;
  g_blocks.erase(it);
  return ok;
}

// ------------------------------------------------------------------ Python API
PyObject* py_set_tag(PyObject*, PyObject* args) {
  const char* t;
  if (!PyArg_ParseTuple(args, "s", &t)) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  g_tag = t;
  Py_RETURN_NONE;
}

PyObject* py_get_tag(PyObject*, PyObject*) {
  std::lock_guard<std::mutex> lk(g_mu);
  return PyUnicode_FromString(g_tag.c_str());
}

PyObject* py_use_fake(PyObject*, PyObject* args) {
  int f;
  if (!PyArg_ParseTuple(args, "p", &f)) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_blocks.empty()) {
    PyErr_SetString(PyExc_RuntimeError, "cannot switch driver mode while allocations are live");
    return nullptr;
  }
  g_fake = f != 0;
  Py_RETURN_NONE;
}

PyObject* py_alloc(PyObject*, PyObject* args) {
  unsigned long long size;
  int device;
  if (!PyArg_ParseTuple(args, "Ki", &size, &device)) return nullptr;
  unsigned long long p = do_alloc((size_t)size, device);
  if (!p) {
    PyErr_SetString(PyExc_MemoryError, g_last_error.c_str());
    return nullptr;
  }
  return PyLong_FromUnsignedLongLong(p);
}

PyObject* py_free(PyObject*, PyObject* args) {
  unsigned long long p;
  if (!PyArg_ParseTuple(args, "K", &p)) return nullptr;
  if (!do_free(p)) {
    PyErr_SetString(PyExc_RuntimeError, g_last_error.c_str());
    return nullptr;
  }
  Py_RETURN_NONE;
}

PyObject* py_allocations(PyObject*, PyObject*) {
  std::lock_guard<std::mutex> lk(g_mu);
  PyObject* lst = PyList_New(0);
  for (auto& kv : g_blocks) {
    PyObject* t = Py_BuildValue("(KKisO)", kv.first, (unsigned long long)kv.second.size, kv.second.device,
                                kv.second.tag.c_str(), kv.second.mapped ? Py_True : Py_False);
    PyList_Append(lst, t);
    Py_DECREF(t);
  }
  return lst;
}

PyObject* py_release(PyObject*, PyObject* args) {
  unsigned long long p;
  if (!PyArg_ParseTuple(args, "K", &p)) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_blocks.find(p);
  if (it == g_blocks.end()) {
    PyErr_SetString(PyExc_KeyError, "unknown allocation");
    return nullptr;
  }
  if (!unback_range(p, it->second)) {
    PyErr_SetString(PyExc_RuntimeError, g_last_error.c_str());
    return nullptr;
  }
  Py_RETURN_NONE;
}

PyObject* py_restore(PyObject*, PyObject* args) {
  unsigned long long p;
  if (!PyArg_ParseTuple(args, "K", &p)) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_blocks.find(p);
  if (it == g_blocks.end()) {
    PyErr_SetString(PyExc_KeyError, "unknown allocation");
    return nullptr;
  }
  if (!it->second.mapped && !back_range(p, it->second)) {
    PyErr_SetString(PyExc_MemoryError, g_last_error.c_str());
    return nullptr;
  }
  Py_RETURN_NONE;
}

// copy(ptr, host_ptr, nbytes, to_host): synchronous copy between an allocation and host memory
PyObject* py_copy(PyObject*, PyObject* args) {
  unsigned long long dev, host, n;
  int to_host;
  if (!PyArg_ParseTuple(args, "KKKp", &dev, &host, &n, &to_host)) return nullptr;
  bool ok = true;
  if (g_fake) {
    if (to_host) std::memcpy(reinterpret_cast<void*>(host), reinterpret_cast<void*>(dev), n);
    else std::memcpy(reinterpret_cast<void*>(dev), reinterpret_cast<void*>(host), n);
  } else {
    Py_BEGIN_ALLOW_THREADS
    std::lock_guard<std::mutex> lk(g_mu);
    ok = load_driver() &&
         (to_host ? check(g_drv.memcpyDtoH(reinterpret_cast<void*>(host), (CUdeviceptr)dev, n), "cuMemcpyDtoH")
                  : check(g_drv.memcpyHtoD((CUdeviceptr)dev, reinterpret_cast<const void*>(host), n), "cuMemcpyHtoD"));
    Py_END_ALLOW_THREADS
  }
  if (!ok) {
    PyErr_SetString(PyExc_RuntimeError, g_last_error.c_str());
    return nullptr;
  }
  Py_RETURN_NONE;
}

PyObject* py_stats(PyObject*, PyObject*) {
  std::lock_guard<std::mutex> lk(g_mu);
  unsigned long long mapped = 0, reserved = 0;
  for (auto& kv : g_blocks) {
    reserved += kv.second.size;
    if (kv.second.mapped) mapped += kv.second.size;
  }
  return Py_BuildValue("{s:K,s:K,s:n}", "mapped_bytes", mapped, "reserved_bytes", reserved, "allocations",
                       (Py_ssize_t)g_blocks.size());
}

PyMethodDef kMethods[] = {
    {"set_tag", py_set_tag, METH_VARARGS, "tag for subsequent allocations"},
    {"get_tag", py_get_tag, METH_NOARGS, "current tag"},
    {"use_fake_driver", py_use_fake, METH_VARARGS, "emulate the driver with host memory"},
    {"alloc", py_alloc, METH_VARARGS, "alloc(size, device) -> ptr"},
    {"free", py_free, METH_VARARGS, "free(ptr)"},
    {"allocations", py_allocations, METH_NOARGS, "[(ptr, size, device, tag, mapped)]"},
    {"release", py_release, METH_VARARGS, "drop the physical memory behind ptr"},
    {"restore", py_restore, METH_VARARGS, "back ptr with fresh physical memory"},
    {"copy", py_copy, METH_VARARGS, "copy(ptr, host_ptr, nbytes, to_host)"},
    {"stats", py_stats, METH_NOARGS, "byte counters"},
    {nullptr, nullptr, 0, nullptr}};

PyModuleDef kModule = {PyModuleDef_HEAD_INIT, "_b200_cumem", "sleep-mode VMM allocator", -1, kMethods};

}  // namespace

// Entry points for torch.cuda.memory.CUDAPluggableAllocator.
extern "C" {
__attribute__((visibility("default"))) void* b200_cumem_malloc(ssize_t size, int device, void* /*stream*/) {
  return reinterpret_cast<void*>(do_alloc((size_t)size, device));
}
__attribute__((visibility("default"))) void b200_cumem_free(void* ptr, ssize_t /*size*/, int /*device*/, void* /*stream*/) {
  do_free(reinterpret_cast<unsigned long long>(ptr));
}
}

PyMODINIT_FUNC PyInit__b200_cumem(void) { return PyModule_Create(&kModule); }
