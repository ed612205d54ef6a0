// Host side of the split-context tensor-core decode kernel (decode_mma_kernel.cuh):
// eligibility of a cache layout for the tensor-core kernels, TMA tensor maps (cached),
// the device status word, and the dispatch to the instantiation of the K/V mode pair
// (compiled in decode_mma_inst_*.cu).

#include <cuda.h>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <type_traits>
#include <vector>

#include "decode_mma_common.cuh"

namespace knlp {

// Set by a kernel whose bounded barrier wait ran out (never expected); read and
// cleared by knlp_b200_debug_status().
__device__ int g_decode_status = 0;

// Device address of the status word on the current device (looked up once per device).
int* decode_status_ptr() {
  constexpr int kMaxDevices = 64;
  static std::atomic<int*> cached[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return nullptr;
  }
  int* p = cached[dev].load(std::memory_order_acquire);
  if (p) return p;
  void* q = nullptr;
  if (cudaGetSymbolAddress(&q, g_decode_status) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  cached[dev].store(static_cast<int*>(q), std::memory_order_release);
  return static_cast<int*>(q);
}

int read_and_clear_decode_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_decode_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int));
  return v;
}

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point (no libcuda link).
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      p = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

bool encode(CUtensorMap* m, void* base, int rank, const cuuint64_t* dims,
            const cuuint64_t* strides, const cuuint32_t* box, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint32_t ones[5] = {1, 1, 1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, static_cast<cuuint32_t>(rank), base, dims, strides,
            box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Codes of one plane in 128-byte rows (see TmaMaps).  Returns 0 if the layout does not
// fit, 1 for the wide form, 2 for the narrow form.
int codes_map(CUtensorMap* m, const Plane& p, int row_bytes, int hpb, const DecodeArgs& a) {
  if (p.cs[2] != row_bytes) return 0;  // the heads of a token must be contiguous
  const int64_t token_bytes = static_cast<int64_t>(a.n_kv_heads) * row_bytes;
  const int seg = hpb * row_bytes;  // the CTA's share of a token row
  if (seg >= 128) {
    if (seg % 128 || token_bytes % 128 || p.cs[1] < token_bytes || p.cs[0] < p.cs[1]) return 0;
    // dimension order (128 bytes, tokens of a page, 128-byte columns of a token row,
    // blocks): one box brings ALL the CTA's columns of 16 tokens, column-major in
    // shared memory ([column][token][128 bytes])
    const cuuint64_t dims[4] = {128, static_cast<cuuint64_t>(a.block_size),
                                static_cast<cuuint64_t>(token_bytes / 128),
                                static_cast<cuuint64_t>(a.num_blocks)};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(p.cs[1]), 128,
                                   static_cast<cuuint64_t>(p.cs[0])};
    const cuuint32_t box[4] = {128, 16, static_cast<cuuint32_t>(seg / 128), 1};
    return encode(m, p.codes, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B) ? 1 : 0;
  }
  // narrow: the CTA holds every head and consecutive tokens are adjacent in memory
  if (hpb != a.n_kv_heads || p.cs[1] != seg) return 0;
  const int64_t page_bytes = static_cast<int64_t>(a.block_size) * seg;
  if (page_bytes % 128 || p.cs[0] < page_bytes) return 0;
  if ((16 * seg) % 1024) return 0;  // a tile must start on the swizzle's 1 KB period
  const cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(page_bytes / 128),
                              static_cast<cuuint64_t>(a.num_blocks)};
  const cuuint64_t strides[2] = {128, static_cast<cuuint64_t>(p.cs[0])};
  const cuuint32_t box[3] = {128, static_cast<cuuint32_t>(16 * seg / 128), 1};
  return encode(m, p.codes, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B) ? 2 : 0;
}

// One scale / zero array as bytes.  merged = false: (all heads of a token, tokens of a
// page, blocks), box = the CTA's heads x 16 tokens.  merged = true (the CTA holds every
// head and the rows of consecutive tokens are adjacent): (4-byte words of a page, 1,
// blocks), box = the words of 16 tokens in one run.
bool scale_map(CUtensorMap* m, __half* base, const int64_t st[3], int sb, int hpb, bool merged,
               const DecodeArgs& a) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint32_t ones[3] = {1, 1, 1};
  if (merged) {
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(a.block_size) * hpb * sb / 4, 1,
                                static_cast<cuuint64_t>(a.num_blocks)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(st[0]) * 2,
                                   static_cast<cuuint64_t>(st[0]) * 2};
    const cuuint32_t box[3] = {static_cast<cuuint32_t>(16 * hpb * sb / 4), 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, base, dims, strides, box, ones,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
           CUDA_SUCCESS;
  }
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(a.n_kv_heads) * sb,
                              static_cast<cuuint64_t>(a.block_size),
                              static_cast<cuuint64_t>(a.num_blocks)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(st[1]) * 2,
                                 static_cast<cuuint64_t>(st[0]) * 2};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(hpb * sb), 16, 1};
  return encode(m, base, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

// Which scale layout the TMA path can take: 0 none, 1 per-token rows, 2 merged.
int scale_layout(const int64_t st[3], const void* base, int ng, int sb, int hpb,
                 const DecodeArgs& a) {
  if (reinterpret_cast<uintptr_t>(base) % 16 || st[2] != ng) return 0;
  if (hpb == a.n_kv_heads && st[1] == static_cast<int64_t>(hpb) * ng && (st[0] * 2) % 16 == 0 &&
      st[0] >= static_cast<int64_t>(a.block_size) * hpb * ng && 16 * hpb * sb <= 1024)
    return 2;
  if ((hpb * sb) % 16 == 0 && (st[1] * 2) % 16 == 0 && (st[0] * 2) % 16 == 0 &&
      st[1] >= static_cast<int64_t>(a.n_kv_heads) * ng && st[0] >= st[1])
    return 1;
  return 0;
}

// Tensor maps are cached by what determines them, so steady-state decode steps do
// not call the driver.
struct MapKey {
  const void* ptrs[6];
  int64_t strides[6][3];
  int64_t num_blocks;
  int n_kv_heads, head_dim, block_size, k_mode, v_mode, hpb;
};

bool build_maps(const DecodeArgs& a, int hpb, TmaMaps* out) {
  if (a.block_size < 16) return false;
  if (a.v.mode == KNLP_KV_INT8_G32) return false;  // INT8 V is staged with cp.async only
  const int ng = a.head_dim / 32, sb = ng * 2;
  // every TMA destination (a scale box is 16 tokens x hpb heads) must be 128-byte aligned
  if ((16 * sb * hpb) % 128) return false;
  const bool asym_k = a.k.mode == KNLP_KV_INT4_ASYM, asym_v = a.v.mode == KNLP_KV_INT4_ASYM;
  const int lay = scale_layout(a.k.ss, a.k.scales, ng, sb, hpb, a);
  if (lay == 0) return false;
  if (scale_layout(a.v.ss, a.v.scales, ng, sb, hpb, a) != lay) return false;
  if (asym_k && scale_layout(a.k.zs, a.k.zeros, ng, sb, hpb, a) != lay) return false;
  if (asym_v && scale_layout(a.v.zs, a.v.zeros, ng, sb, hpb, a) != lay) return false;

  MapKey key;
  std::memset(&key, 0, sizeof(key));
  const void* ptrs[6] = {a.k.codes, a.v.codes, a.k.scales, a.k.zeros, a.v.scales, a.v.zeros};
  const int64_t* sts[6] = {a.k.cs, a.v.cs, a.k.ss, a.k.zs, a.v.ss, a.v.zs};
  for (int i = 0; i < 6; ++i) {
    key.ptrs[i] = ptrs[i];
    for (int j = 0; j < 3; ++j) key.strides[i][j] = sts[i][j];
  }
  key.num_blocks = a.num_blocks;
  key.n_kv_heads = a.n_kv_heads;
  key.head_dim = a.head_dim;
  key.block_size = a.block_size;
  key.k_mode = a.k.mode;
  key.v_mode = a.v.mode;
  key.hpb = hpb;

  static std::mutex mu;
  static std::vector<std::pair<MapKey, TmaMaps>> cache;
  std::lock_guard<std::mutex> lock(mu);
  for (const auto& e : cache) {
    if (std::memcmp(&e.first, &key, sizeof(key)) == 0) {
      *out = e.second;
      return true;
    }
  }
  TmaMaps m;
  std::memset(&m, 0, sizeof(m));
  const bool merged = lay == 2;
  m.scale_merged = merged ? 1 : 0;
  const int kb = a.k.mode == KNLP_KV_INT8_G32 ? a.head_dim : a.head_dim / 2;
  const int kform = codes_map(&m.k, a.k, kb, hpb, a);
  const int vform = codes_map(&m.v, a.v, a.head_dim / 2, hpb, a);  // (INT8 V never gets here)
  if (kform == 0 || vform == 0) return false;
  m.k_narrow = kform == 2;
  m.v_narrow = vform == 2;
  if (!scale_map(&m.ks, a.k.scales, a.k.ss, sb, hpb, merged, a)) return false;
  if (!scale_map(&m.vs, a.v.scales, a.v.ss, sb, hpb, merged, a)) return false;
  m.kz = m.ks;
  m.vz = m.vs;
  if (asym_k && !scale_map(&m.kz, a.k.zeros, a.k.zs, sb, hpb, merged, a)) return false;
  if (asym_v && !scale_map(&m.vz, a.v.zeros, a.v.zs, sb, hpb, merged, a)) return false;
  if (cache.size() >= 64) cache.erase(cache.begin());
  cache.emplace_back(key, m);
  *out = m;
  return true;
}

}  // namespace

// Defined in decode_mma_inst_*.cu (one translation unit per mode pair).
template <int KMODE, int VMODE>
int launch_mma_pair(const DecodeArgs& a, const MmaParams& mp, bool split, const TmaMaps* tm,
                    cudaStream_t st);
#define KNLP_DECL_PAIR(K, V)                                                              \
  extern template int launch_mma_pair<K, V>(const DecodeArgs&, const MmaParams&, bool,   \
                                            const TmaMaps*, cudaStream_t)
KNLP_DECL_PAIR(KNLP_KV_INT4_ASYM, KNLP_KV_INT4_ASYM);
KNLP_DECL_PAIR(KNLP_KV_INT4_SYM, KNLP_KV_INT4_SYM);
KNLP_DECL_PAIR(KNLP_KV_INT8_G32, KNLP_KV_INT4_ASYM);
KNLP_DECL_PAIR(KNLP_KV_INT8_G32, KNLP_KV_INT4_SYM);
KNLP_DECL_PAIR(KNLP_KV_INT8_G32, KNLP_KV_INT8_G32);
#undef KNLP_DECL_PAIR

namespace {

int launch_modes(const DecodeArgs& a, const MmaParams& mp, bool split, const TmaMaps* tm,
                 cudaStream_t st) {
  const int km = a.k.mode, vm = a.v.mode;
  if (km == KNLP_KV_INT4_ASYM && vm == KNLP_KV_INT4_ASYM)
    return launch_mma_pair<KNLP_KV_INT4_ASYM, KNLP_KV_INT4_ASYM>(a, mp, split, tm, st);
  if (km == KNLP_KV_INT4_SYM && vm == KNLP_KV_INT4_SYM)
    return launch_mma_pair<KNLP_KV_INT4_SYM, KNLP_KV_INT4_SYM>(a, mp, split, tm, st);
  if (km == KNLP_KV_INT8_G32 && vm == KNLP_KV_INT4_ASYM)
    return launch_mma_pair<KNLP_KV_INT8_G32, KNLP_KV_INT4_ASYM>(a, mp, split, tm, st);
  if (km == KNLP_KV_INT8_G32 && vm == KNLP_KV_INT4_SYM)
    return launch_mma_pair<KNLP_KV_INT8_G32, KNLP_KV_INT4_SYM>(a, mp, split, tm, st);
  if (km == KNLP_KV_INT8_G32 && vm == KNLP_KV_INT8_G32)
    return launch_mma_pair<KNLP_KV_INT8_G32, KNLP_KV_INT8_G32>(a, mp, split, tm, st);
  return 1;  // other combinations go to the generic kernel
}

bool aligned(const void* p, uintptr_t n) { return reinterpret_cast<uintptr_t>(p) % n == 0; }

// What the cp.async loader needs: 32-bit strides, 16-byte aligned pieces, the heads of
// a token adjacent in memory (codes and scales), and scale rows that can be cut into
// 16-byte pieces (a token's row of the CTA's heads is a multiple of 16 bytes, or the CTA
// holds every head and consecutive tokens are adjacent).
bool scale_array_ok(const __half* base, const int64_t st[3], int ng, int hpb, int n_kv_heads) {
  constexpr int64_t kMax = 0x3fffffff;
  if (!aligned(base, 16) || st[2] != ng) return false;
  for (int i = 0; i < 2; ++i)
    if (st[i] < 0 || st[i] > kMax || (st[i] * 2) % 16 != 0 && i == 0) return false;
  const int tb = hpb * ng * 2;  // bytes of one token's row
  if (tb % 16 == 0) return (st[1] * 2) % 16 == 0;
  return hpb == n_kv_heads && st[1] * 2 == tb && 16 % tb == 0;
}

bool plane_ok(const Plane& p, int head_dim, int row_bytes, int hpb, int n_kv_heads) {
  constexpr int64_t kMax = 0x7fffffff;
  if (!aligned(p.codes, 16) || p.cs[2] != row_bytes) return false;
  for (int i = 0; i < 2; ++i)
    if (p.cs[i] % 16 || p.cs[i] < 0 || p.cs[i] > kMax) return false;
  const int ng = head_dim / 32;
  if (p.mode == KNLP_KV_F16 || p.mode == KNLP_KV_BF16) return true;  // no scale rows
  if (!scale_array_ok(p.scales, p.ss, ng, hpb, n_kv_heads)) return false;
  if (p.zeros && !scale_array_ok(p.zeros, p.zs, ng, hpb, n_kv_heads)) return false;
  return true;
}

}  // namespace

// Shape and layout test shared by the tensor-core kernels: 0 = they can take the
// call (hpb_log2 / page_log2 filled in), 1 = only the generic kernel can.
int decode_mma_layout(const DecodeArgs& a, int* hpb_log2_out, int* page_log2_out) {
  if (a.head_dim != 64 && a.head_dim != 128) return 1;
  if (a.n_q_heads % a.n_kv_heads) return 1;
  const int n_rep = a.n_q_heads / a.n_kv_heads;
  if (n_rep > 8) return 1;
  if (a.block_size & (a.block_size - 1)) return 1;  // pages must be a power of two
  if (a.num_blocks > 0x7fffffff) return 1;
  int hpb_log2 = kWarpsLog;
  while (hpb_log2 > 0 && (a.n_kv_heads % (1 << hpb_log2))) --hpb_log2;
  const int hpb = 1 << hpb_log2;
  const int kb = (a.k.mode == KNLP_KV_F16 || a.k.mode == KNLP_KV_BF16) ? 2 * a.head_dim
                 : a.k.mode == KNLP_KV_INT8_G32                           ? a.head_dim
                                                                          : a.head_dim / 2;
  if (!plane_ok(a.k, a.head_dim, kb, hpb, a.n_kv_heads) ||
      !plane_ok(a.v, a.head_dim, a.v.mode == KNLP_KV_INT8_G32 ? a.head_dim : a.head_dim / 2, hpb,
                a.n_kv_heads))
    return 1;
  int page_log2 = 0;
  while ((1 << page_log2) < a.block_size) ++page_log2;
  *hpb_log2_out = hpb_log2;
  *page_log2_out = page_log2;
  return 0;
}

int launch_decode_mma(const DecodeArgs& a, bool allow_tma, bool debug_stall, cudaStream_t st) {
  MmaParams mp{};
  mp.debug_stall = debug_stall ? 1 : 0;
  if (decode_mma_layout(a, &mp.hpb_log2, &mp.page_log2)) return 1;
  // the page-id ring of the kernel holds 16 ids per stage; a stage is (warps / heads per
  // CTA) * 16 tokens, so blocks of 1 or 2 tokens can need more: the generic kernel takes those
  if ((kDecodeWarps >> mp.hpb_log2) * 16 > 16 * a.block_size) return 1;
  mp.status = decode_status_ptr();
  if (!mp.status) return KNLP_ERR_NO_DEVICE;
  const int hpb = 1 << mp.hpb_log2;
  const bool split = a.n_q_heads / a.n_kv_heads <= 4;
  TmaMaps tm;
  const bool use_tma = allow_tma && build_maps(a, hpb, &tm);
  const TmaMaps* tmp = use_tma ? &tm : nullptr;
  return launch_modes(a, mp, split, tmp, st);
}

}  // namespace knlp
