// Runtime part of the C ABI: device binding, buffers, copies, error text.
// Stands where backends/nvidia/runtime/runtime.go stands in the reference (Init,
// EnsureContext, Malloc, Buffer.Upload/Download/Free, Sync).
#include <dlfcn.h>
#include <stdarg.h>
#include <string.h>

#include <atomic>

#include "goph_internal.cuh"

namespace goph {

static DeviceState g_dev[kMaxDevices];
static thread_local char g_err[512] = "";

static Options g_opt;

// Driver contexts adopted through goph_init_current_context (nullptr: the device's primary
// context, bound through the runtime).  The reference creates its own context with cuCtxCreate
// (backends/nvidia/runtime/runtime.go:247) and allocates every buffer in it, so a drop-in has to
// launch in that context and leave it current on the calling thread.
static void* g_ctx[kMaxDevices] = {};
typedef int (*CtxGetCurrent)(void**);
typedef int (*CtxSetCurrent)(void*);
typedef int (*CtxGetDevice)(int*);
static CtxGetCurrent p_ctx_get_current = nullptr;
static CtxSetCurrent p_ctx_set_current = nullptr;
static CtxGetDevice p_ctx_get_device = nullptr;

// The driver library is opened at run time (no link-time dependency, as the reference's purego binding).
static bool load_driver() {
  if (p_ctx_set_current) return true;
  void* h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
  if (!h) return false;
  p_ctx_get_current = (CtxGetCurrent)dlsym(h, "cuCtxGetCurrent");
  p_ctx_get_device = (CtxGetDevice)dlsym(h, "cuCtxGetDevice");
  p_ctx_set_current = (CtxSetCurrent)dlsym(h, "cuCtxSetCurrent");
  return p_ctx_get_current && p_ctx_get_device && p_ctx_set_current;
}

DeviceState& device_state(int device) { return g_dev[device]; }
static std::atomic<unsigned long long> g_launches{0};
void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

Options& options() { return g_opt; }

void clear_error() { g_err[0] = 0; }

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof g_err, fmt, ap);
  va_end(ap);
  return code;
}

int fail_cuda(cudaError_t e, const char* what) {
  snprintf(g_err, sizeof g_err, "CUDA error %d (%s: %s) in %s", (int)e, cudaGetErrorName(e),
           cudaGetErrorString(e), what);
  cudaGetLastError();  // clear the sticky-free error slot for the next call
  return e == cudaErrorMemoryAllocation ? GOPH_E_NOMEM : GOPH_E_CUDA;
}

int use_device(int device) {
  if (device < 0 || device >= kMaxDevices) return fail(GOPH_E_INVALID, "device %d out of range", device);
  if (!g_dev[device].ready) return fail(GOPH_E_NOINIT, "goph_init(%d) has not been called", device);
  if (g_ctx[device]) {
    // an adopted context: make it current (calls may come from any OS thread), the runtime follows it
    int rc = p_ctx_set_current(g_ctx[device]);
    if (rc != 0) return fail(GOPH_E_CUDA, "cuCtxSetCurrent failed with CUresult %d", rc);
    return GOPH_OK;
  }
  GOPH_CUDA(cudaSetDevice(device));
  return GOPH_OK;
}

}  // namespace goph

using namespace goph;

GOPH_API int goph_init(int device) {
  clear_error();
  if (device < 0 || device >= kMaxDevices) return fail(GOPH_E_INVALID, "device %d out of range", device);
  int n = 0;
  GOPH_CUDA(cudaGetDeviceCount(&n));
  if (device >= n) return fail(GOPH_E_INVALID, "device %d not present (%d visible)", device, n);
  DeviceState& st = device_state(device);
  if (st.ready && g_ctx[device])
    return fail(GOPH_E_INVALID, "device %d is already bound to an adopted context (goph_init_current_context)", device);
  GOPH_CUDA(cudaSetDevice(device));
  GOPH_CUDA(cudaFree(0));
  if (st.ready) return GOPH_OK;
  cudaDeviceProp prop;
  GOPH_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(GOPH_E_UNSUPPORTED, "device %d is sm_%d%d; this library holds sm_100a code only", device,
                prop.major, prop.minor);
  st.sm_count = prop.multiProcessorCount;
  st.max_smem_optin = (int)prop.sharedMemPerBlockOptin;
  st.ready = true;
  return GOPH_OK;
}

GOPH_API int goph_init_current_context(int* out_device) {
  clear_error();
  if (!out_device) return fail(GOPH_E_INVALID, "goph_init_current_context: nil result pointer");
  *out_device = -1;
  if (!load_driver()) return fail(GOPH_E_CUDA, "goph_init_current_context: libcuda.so.1 cannot be opened");
  void* ctx = nullptr;
  int rc = p_ctx_get_current(&ctx);
  if (rc != 0 || !ctx)
    return fail(GOPH_E_INVALID, "goph_init_current_context: no driver context is current on this thread (CUresult %d)", rc);
  int device = -1;
  rc = p_ctx_get_device(&device);
  if (rc != 0 || device < 0 || device >= kMaxDevices)
    return fail(GOPH_E_INVALID, "goph_init_current_context: cuCtxGetDevice gave device %d (CUresult %d)", device, rc);
  DeviceState& st = device_state(device);
  if (st.ready && g_ctx[device] != ctx)
    return fail(GOPH_E_INVALID, "device %d is already bound to %s context: a device serves one context per process", device,
                g_ctx[device] ? "another adopted" : "its primary");
  if (st.ready) {
    *out_device = device;
    return GOPH_OK;
  }
  cudaDeviceProp prop;
  GOPH_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(GOPH_E_UNSUPPORTED, "device %d is sm_%d%d; this library holds sm_100a code only", device, prop.major, prop.minor);
  st.sm_count = prop.multiProcessorCount;
  st.max_smem_optin = (int)prop.sharedMemPerBlockOptin;
  g_ctx[device] = ctx;
  st.ready = true;
  *out_device = device;
  return GOPH_OK;
}

GOPH_API int goph_launch_count(uint64_t* out_count) {
  clear_error();
  if (!out_count) return fail(GOPH_E_INVALID, "goph_launch_count: null result");
  *out_count = g_launches.load(std::memory_order_relaxed);
  return GOPH_OK;
}

GOPH_API int goph_set_option(const char* name, int value) {
  clear_error();
  if (!name) return fail(GOPH_E_INVALID, "goph_set_option: nil name");
  Options& o = options();
  bool rows_ok = value == 0 || value == 1 || value == 2 || value == 4;
  if (!strcmp(name, "pdl")) {
    o.pdl = value != 0;
  } else if (!strcmp(name, "mlx_fuse")) {
    o.mlx_fuse = value ? 1 : 0;
  } else if (!strcmp(name, "mlx_ctas_per_sm")) {
    if (value < 0 || value > 8) return fail(GOPH_E_INVALID, "mlx_ctas_per_sm=%d not in 0..8", value);
    o.mlx_ctas_per_sm = value;
  } else if (!strcmp(name, "gguf_layout")) {
    if (value < 0 || value > 2) return fail(GOPH_E_INVALID, "gguf_layout=%d not in 0..2", value);
    o.gguf_layout = value;
  } else if (!strcmp(name, "fp8_layout")) {
    if (value < 0 || value > 2) return fail(GOPH_E_INVALID, "fp8_layout=%d not in 0..2", value);
    o.fp8_layout = value;
  } else if (!strcmp(name, "mlx_layout")) {
    if (value < 0 || value > 2) return fail(GOPH_E_INVALID, "mlx_layout=%d not in 0..2", value);
    o.mlx_layout = value;
  } else if (!strcmp(name, "moe_fused")) {
    o.moe_fused = value ? 1 : 0;
  } else if (!strcmp(name, "moe_rows")) {
    if (value != 0 && value != 2 && value != 4) return fail(GOPH_E_INVALID, "moe_rows=%d not 0, 2 or 4", value);
    o.moe_rows = value;
  } else if (!strcmp(name, "mlx_cluster")) {
    o.mlx_cluster = value ? 1 : 0;
  } else if (!strcmp(name, "fp8_convert")) {
    o.fp8_convert = value ? 1 : 0;
  } else if (!strcmp(name, "mlx_chunks")) {
    if (value < 0 || value > 2) return fail(GOPH_E_INVALID, "mlx_chunks=%d not in 0..2", value);
    o.mlx_chunks = value;
  } else if (!strcmp(name, "mlx_splits")) {
    if (value < 0 || value > 64) return fail(GOPH_E_INVALID, "mlx_splits=%d not in 0..64", value);
    o.mlx_splits = value;
  } else if (!strcmp(name, "mlx_digits")) {
    if (value != 3 && value != 4) return fail(GOPH_E_INVALID, "mlx_digits=%d not 3 or 4", value);
    o.mlx_digits = value;
  } else if (!strcmp(name, "mlx_unpack")) {
    if (value < 0 || value > 2) return fail(GOPH_E_INVALID, "mlx_unpack=%d not in 0..2", value);
    o.mlx_unpack = value;
  } else if (!strcmp(name, "mlx_rows") && rows_ok) {
    o.mlx_rows = value;
  } else if (!strcmp(name, "gguf_rows") && rows_ok) {
    o.gguf_rows = value;
  } else if (!strcmp(name, "fp8_rows") && rows_ok) {
    o.fp8_rows = value;
  } else {
    return fail(GOPH_E_INVALID, "goph_set_option: unknown option or bad value %s=%d", name, value);
  }
  return GOPH_OK;
}

GOPH_API const char* goph_last_error(void) { return g_err; }

GOPH_API int goph_sm_count(int device) {
  if (device < 0 || device >= kMaxDevices || !device_state(device).ready) return 0;
  return device_state(device).sm_count;
}

GOPH_API int goph_malloc(int device, uint64_t bytes, void** out_dev) {
  clear_error();
  if (!out_dev) return fail(GOPH_E_INVALID, "goph_malloc: nil result pointer");
  *out_dev = nullptr;
  if (bytes == 0) return fail(GOPH_E_INVALID, "goph_malloc: zero bytes");
  if (int rc = use_device(device)) return rc;
  GOPH_CUDA(cudaMalloc(out_dev, bytes));
  return GOPH_OK;
}

GOPH_API int goph_free(int device, void* dev) {
  clear_error();
  if (!dev) return GOPH_OK;
  if (int rc = use_device(device)) return rc;
  GOPH_CUDA(cudaFree(dev));
  return GOPH_OK;
}

GOPH_API int goph_upload(int device, void* dst_dev, const void* src_host, uint64_t bytes) {
  clear_error();
  if (bytes == 0) return GOPH_OK;
  if (!dst_dev || !src_host) return fail(GOPH_E_INVALID, "goph_upload: nil pointer");
  if (int rc = use_device(device)) return rc;
  GOPH_CUDA(cudaMemcpy(dst_dev, src_host, bytes, cudaMemcpyHostToDevice));
  return GOPH_OK;
}

GOPH_API int goph_download(int device, void* dst_host, const void* src_dev, uint64_t bytes) {
  clear_error();
  if (bytes == 0) return GOPH_OK;
  if (!dst_host || !src_dev) return fail(GOPH_E_INVALID, "goph_download: nil pointer");
  if (int rc = use_device(device)) return rc;
  GOPH_CUDA(cudaMemcpy(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost));
  return GOPH_OK;
}

GOPH_API int goph_memset(int device, void* dst_dev, int byte, uint64_t bytes) {
  clear_error();
  if (bytes == 0) return GOPH_OK;
  if (!dst_dev) return fail(GOPH_E_INVALID, "goph_memset: nil pointer");
  if (int rc = use_device(device)) return rc;
  GOPH_CUDA(cudaMemset(dst_dev, byte, bytes));
  return GOPH_OK;
}

GOPH_API int goph_sync(int device) {
  clear_error();
  if (int rc = use_device(device)) return rc;
  GOPH_CUDA(cudaDeviceSynchronize());
  return GOPH_OK;
}
