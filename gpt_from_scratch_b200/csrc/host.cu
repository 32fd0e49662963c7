// Host-side runtime shared by all kernels: tensor-map encoding (driver entry point
// fetched at run time so the library links against cudart only), a small tensor-map
// cache, the per-device status words and device properties.
#include <cstdlib>
#include <mutex>
#include <unordered_map>
#include <vector>
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace gfs_host {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int encode_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                     const uint32_t* box) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bdim[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i];
  }
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), gdim, gstr, bdim, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // a driver-API call on a thread that has made no runtime call yet (e.g. the first operator an
    // autograd worker thread runs): bind the device's primary context to the thread and retry
    cudaFree(nullptr);
    r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), gdim, gstr, bdim, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[gfs] cuTensorMapEncodeTiled failed: %d (rank %d base %p dims %llu %llu box %u %u)\n", (int)r,
            rank, base, (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 0), box[0],
            rank > 1 ? box[1] : 0);
    return -2;
  }
  return 0;
}

struct Key2D {
  const void* base;
  uint64_t rows, cols, ld;
  uint32_t br, bc;
  bool operator==(const Key2D& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && br == o.br && bc == o.bc;
  }
};
struct Key2DHash {
  size_t operator()(const Key2D& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h ^= k.rows * 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
    h ^= k.cols * 0xc2b2ae3d27d4eb4full + (h << 6) + (h >> 2);
    h ^= k.ld * 0x165667b19e3779f9ull + (h << 6) + (h >> 2);
    h ^= (static_cast<size_t>(k.br) << 32 | k.bc) + (h << 6) + (h >> 2);
    return h;
  }
};

const CUtensorMap* tmap_2d_cached(const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                                  uint32_t box_rows, uint32_t box_cols) {
  static std::mutex mu;
  static std::unordered_map<Key2D, CUtensorMap*, Key2DHash> cache;
  Key2D key{base, rows, cols, ld_elems, box_rows, box_cols};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  if (cache.size() > 8192) {  // bounded: drop everything, maps are cheap to rebuild
    for (auto& kv : cache) delete kv.second;
    cache.clear();
  }
  CUtensorMap* m = new CUtensorMap;
  uint64_t dims[2] = {cols, rows};
  uint64_t strides[2] = {2, ld_elems * 2};
  uint32_t box[2] = {box_cols, box_rows};
  if (encode_tmap_bf16(m, base, 2, dims, strides, box) != 0) {
    delete m;
    return nullptr;
  }
  cache.emplace(key, m);
  return m;
}

struct KeyND {
  const void* base;
  int rank;
  uint64_t dims[4];
  uint64_t strides[4];
  uint32_t box[4];
  bool operator==(const KeyND& o) const { return memcmp(this, &o, sizeof(KeyND)) == 0; }
};
struct KeyNDHash {
  size_t operator()(const KeyND& k) const {
    const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
    size_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(KeyND) / 8; ++i) h = (h ^ w[i]) * 1099511628211ull;
    return h;
  }
};

// Cached tensor map of rank <= 4 (dims/strides innermost first, strides in bytes).
const CUtensorMap* tmap_nd_cached(const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                                  const uint32_t* box) {
  static std::mutex mu;
  static std::unordered_map<KeyND, CUtensorMap*, KeyNDHash> cache;
  KeyND key;
  memset(&key, 0, sizeof(key));
  key.base = base;
  key.rank = rank;
  for (int i = 0; i < rank; ++i) {
    key.dims[i] = dims[i];
    key.strides[i] = strides_bytes[i];
    key.box[i] = box[i];
  }
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  if (cache.size() > 8192) {
    for (auto& kv : cache) delete kv.second;
    cache.clear();
  }
  CUtensorMap* m = new CUtensorMap;
  if (encode_tmap_bf16(m, base, rank, dims, strides_bytes, box) != 0) {
    delete m;
    return nullptr;
  }
  cache.emplace(key, m);
  return m;
}

uint32_t* status_words() {
  static std::mutex mu;
  static uint32_t* per_dev[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  if (per_dev[dev] == nullptr) {
    uint32_t* p = nullptr;
    if (cudaMalloc(&p, 64 * sizeof(uint32_t)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 64 * sizeof(uint32_t));
    per_dev[dev] = p;
  }
  return per_dev[dev];
}

bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = std::getenv("GFS_PDL");
    on = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

int sm_count() {
  static int per_dev[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (per_dev[dev] == 0) {
    cudaDeviceGetAttribute(&per_dev[dev], cudaDevAttrMultiProcessorCount, dev);
  }
  return per_dev[dev];
}

}  // namespace gfs_host

extern "C" {

// Reads (and optionally clears) the status words of the current device. Synchronises
// the device. out must hold 2 uint32: [code, detail]. Returns the code.
// Number of counters in a flag array; the array handed to the fused collectives must hold twice
// as many uint32 words (counters, then their base words: see common.cuh).
int gfs_flag_slots() { return static_cast<int>(gfs::FLAG_SLOTS); }

int gfs_read_status(uint32_t* out, int clear) {
  uint32_t* p = gfs_host::status_words();
  uint32_t h[2] = {0, 0};
  if (p == nullptr) return -1;
  if (cudaMemcpy(h, p, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (clear && h[0] != 0) cudaMemset(p, 0, 2 * sizeof(uint32_t));
  if (out != nullptr) {
    out[0] = h[0];
    out[1] = h[1];
  }
  return static_cast<int>(h[0]);
}

int gfs_sm_count() { return gfs_host::sm_count(); }

const char* gfs_last_cuda_error() { return cudaGetErrorString(cudaGetLastError()); }

}  // extern "C"
