// Host-side plumbing shared by every entry point: error strings, the device status word, the
// tensor-map encoder lookup and device properties.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include <mutex>

#include "common.cuh"

namespace dflash {
namespace {
thread_local char g_err[512] = "";
__device__ int g_device_status = 0;
std::mutex g_mu;
int* g_status_ptr[64] = {};
int g_sm_count[64] = {};
tensormap_encode_fn g_encoder = nullptr;
bool g_encoder_tried = false;
int g_pdl = -1;                        // -1: not decided yet (environment DFLASH_PDL, default on)
thread_local int g_pdl_skip = 0;       // launches of this thread that must be plain (fully serialised)
}  // namespace

bool pdl_enabled_for_next_launch() {
  if (g_pdl < 0) {
    const char* e = getenv("DFLASH_PDL");
    g_pdl = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  if (g_pdl_skip > 0) {
    --g_pdl_skip;
    return false;
  }
  return g_pdl == 1;
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int* device_error_word(int device) {
  std::lock_guard<std::mutex> lk(g_mu);
  int* p = g_status_ptr[device & 63];
  if (p == nullptr) {
    if (cudaGetSymbolAddress((void**)&p, g_device_status) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    g_status_ptr[device & 63] = p;
  }
  return p;
}

tensormap_encode_fn get_tensormap_encoder() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_encoder_tried) {
    g_encoder_tried = true;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encoder = (tensormap_encode_fn)fn;
    else {
      cudaGetLastError();
      set_error("cuTensorMapEncodeTiled is not available from this driver");
    }
  }
  return g_encoder;
}

int sm_count(int device) {
  std::lock_guard<std::mutex> lk(g_mu);
  int& c = g_sm_count[device & 63];
  if (c == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || v <= 0) {
      cudaGetLastError();
      v = 148;  // B200; only reached when planning without a device (host-side tests)
    }
    c = v;
  }
  return c;
}
}  // namespace dflash

extern "C" int dflash_version(void) { return 100; }

extern "C" void dflash_set_pdl(int on) { dflash::g_pdl = on ? 1 : 0; }
extern "C" int dflash_get_pdl(void) {
  if (dflash::g_pdl < 0) {
    const char* e = getenv("DFLASH_PDL");
    dflash::g_pdl = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return dflash::g_pdl;
}
extern "C" void dflash_pdl_plain_next(int launches) { dflash::g_pdl_skip = launches > 0 ? launches : 0; }

extern "C" const char* dflash_last_error_string(void) { return dflash::g_err; }

extern "C" int dflash_device_error(int device) {
  int prev = 0;
  if (cudaGetDevice(&prev) != cudaSuccess) { cudaGetLastError(); return 0; }
  cudaSetDevice(device);
  int* p = dflash::device_error_word(device);
  int v = 0;
  if (p != nullptr) {
    cudaDeviceSynchronize();
    cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
    if (v != 0) cudaMemset(p, 0, sizeof(int));
  }
  cudaSetDevice(prev);
  return v;
}
