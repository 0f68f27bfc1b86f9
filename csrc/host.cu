// Status word, error text and the TMA tensor-map cache.
#include "host.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace b2 {

__device__ int g_status_word[4];

static char g_error_text[512] = {0};
static std::mutex g_mu;

static int g_device = -1;

void ensure_thread_context() {
  thread_local int bound = -2;
  if (bound == g_device) return;
  if (g_device >= 0) {
    cudaSetDevice(g_device);
  } else {
    cudaFree(nullptr);  // binds the runtime's default device and creates / attaches its context
  }
  bound = g_device;
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error_text, sizeof(g_error_text), fmt, ap);
  va_end(ap);
}

int* status_ptr() {
  ensure_thread_context();
  static int* ptrs[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) {
      set_error("cudaGetSymbolAddress(status) failed");
      return nullptr;
    }
    cudaMemset(p, 0, sizeof(int) * 4);
    ptrs[dev] = static_cast<int*>(p);
  }
  return ptrs[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess || p == nullptr) {
    set_error("cuTensorMapEncodeTiled entry point unavailable");
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

struct MapKey {
  uint64_t w[12];
  bool operator==(const MapKey& o) const { return memcmp(w, o.w, sizeof(w)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    for (int i = 0; i < 12; ++i) {
      h ^= k.w[i];
      h *= 1099511628211ull;
    }
    return static_cast<size_t>(h);
  }
};

// Entries are heap-allocated and never move, so returned pointers stay valid.
static std::unordered_map<MapKey, CUtensorMap*, MapKeyHash> g_maps;

const CUtensorMap* tensor_map_nd_bf16(const void* base, int rank, const uint64_t* dims,
                                      const uint64_t* strides_bytes, const uint32_t* box,
                                      int swizzle) {
  ensure_thread_context();
  MapKey key;
  memset(&key, 0, sizeof(key));
  int dev = 0;
  cudaGetDevice(&dev);
  key.w[0] = reinterpret_cast<uint64_t>(base);
  key.w[1] = (static_cast<uint64_t>(rank) << 32) | (static_cast<uint64_t>(swizzle) << 8) |
             static_cast<uint64_t>(dev);
  for (int i = 0; i < rank; ++i) {
    key.w[2 + i] = dims[i];
    key.w[6 + i] = (i > 0 ? strides_bytes[i - 1] : 0) ^ (static_cast<uint64_t>(box[i]) << 48);
  }
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) return it->second;
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return nullptr;
  if (g_maps.size() > 65536) {  // unbounded growth guard: drop everything, maps are cheap to rebuild
    for (auto& kv : g_maps) delete kv.second;
    g_maps.clear();
  }
  cuuint64_t gdim[4];
  cuuint64_t gstr[3];
  cuuint32_t bx[4];
  cuuint32_t es[4] = {1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
  }
  CUtensorMapSwizzle sw = swizzle == 3   ? CU_TENSOR_MAP_SWIZZLE_128B
                          : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_32B
                                         : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUtensorMap* m = new CUtensorMap;
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank),
                  const_cast<void*>(base), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed: code %d (base %p rank %d dims %llu %llu box %u %u)",
              static_cast<int>(r), base, rank, (unsigned long long)dims[0],
              (unsigned long long)(rank > 1 ? dims[1] : 0), box[0], rank > 1 ? box[1] : 0);
    delete m;
    return nullptr;
  }
  g_maps.emplace(key, m);
  return m;
}

const CUtensorMap* tensor_map_2d_bf16(const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                                      uint32_t box_rows, uint32_t box_cols) {
  uint64_t dims[2] = {cols, rows};
  uint64_t strides[1] = {ld * 2};
  uint32_t box[2] = {box_cols, box_rows};
  return tensor_map_nd_bf16(base, 2, dims, strides, box, 3);
}

}  // namespace b2

// Reads the status word (synchronises the device), clears it, and returns the value.
B2_EXPORT int b2_status_read_and_clear() {
  int* p = b2::status_ptr();
  if (!p) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (v != 0) cudaMemset(p, 0, sizeof(int));
  return v;
}

// One process drives one GPU: the Python side reports torch's current device once at start-up.
B2_EXPORT void b2_set_device(int device) { b2::g_device = device; }

B2_EXPORT const char* b2_last_error() { return b2::g_error_text; }

B2_EXPORT void b2_clear_tensor_maps() {
  std::lock_guard<std::mutex> lock(b2::g_mu);
  for (auto& kv : b2::g_maps) delete kv.second;
  b2::g_maps.clear();
}
