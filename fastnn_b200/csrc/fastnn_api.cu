// C ABI of libfastnn_b200.so (declared in include/fastnn_b200_kernels.h).
//
// Host side of the GEMM path: per-device state, argument checks, the tile / split-K
// planner, tensor-map encoding and kernel launches.  No cuBLAS, no CPU fallback.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <utility>

#include "../../include/fastnn_b200_kernels.h"
#include "gemm_simt.cuh"
#include "gemm_tcgen05.cuh"
#include "gemm_tcgen05_pair.cuh"
#include "attention_tcgen05.cuh"
#include "conv_tcgen05.cuh"
#include "conv_wgrad_tcgen05.cuh"
#include "conv_wgrad_slab_tcgen05.cuh"

namespace {

using fnn::GemmParams;

constexpr int kMaxDevices = 16;
constexpr size_t kMaxDynSmem = 232448;   // 227 KiB, the sm_100 per-CTA limit
constexpr size_t kCkHalfSmem = 112 * 1024;   // two such CTAs share an SM

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct Workspace {
  float* ptr = nullptr;
  size_t bytes = 0;
};

struct DeviceState {
  std::atomic<bool> ready{false};   // set last by fastnn_cuda_init; everything but the workspace
                                    // tables is constant afterwards
  int num_sms = 0;
  int max_clusters = 0;             // co-resident CTA pairs of the pair kernel
  int ck_slots[5] = {0, 0, 0, 0, 0};  // co-resident CTAs of the cluster split-K kernel at cluster
                                    // size 2^i (index 0 unused); 0 = that size cannot launch
  int ck_slots_half[5] = {0, 0, 0, 0, 0};   // the same when a CTA asks for at most kCkHalfSmem
  unsigned int* status = nullptr;   // device word written by a kernel whose wait ran out
  long long spin_budget = 0;        // clock ticks one wait may last
  std::mutex ws_mutex;                            // guards the two tables below
  std::map<cudaStream_t, Workspace> workspaces;   // split-K partials, one per stream
  std::map<cudaStream_t, Workspace> conv_ws;      // im2col matrix + per-image partials of conv dW
  std::map<cudaStream_t, Workspace> attn_ws;      // scores of the composed attention path
};

std::mutex g_mutex;                 // device initialisation only; no GEMM call takes it
DeviceState g_dev[kMaxDevices];
std::atomic<EncodeTiledFn> g_encode{nullptr};
std::atomic<unsigned long long> g_launches{0};

// Kernel-selection override of fastnn_b200_set_policy: per calling thread, so a test or sweep
// that forces a kernel cannot change what another thread's GEMMs run.
struct Policy {
  int policy = 0, block_n = 0, split_k = 0;
};
thread_local Policy t_policy;

// Environment switches, read once per process (first GEMM call).
struct Tunables {
  bool no_chunked = false;      // FASTNN_B200_NO_CHUNKED: per-chunk boxes for MN-major operands
  bool cluster_k_off = false;   // FASTNN_B200_CLUSTER_K=0
  bool pdl = true;              // FASTNN_B200_PDL=0: ordinary launches
  int kb_per_stage = 0;         // FASTNN_B200_KB_PER_STAGE (CTA pairs; 0 = planner)
  int stages = 0;               // FASTNN_B200_STAGES: upper bound on pipeline stages (0 = none)
  int group_m = 0;              // FASTNN_B200_GROUP_M: tile rows per rasterisation group
  int l2 = -1;                  // FASTNN_B200_L2=<C><A><B>: eviction policies of stores and loads
  bool no_wide = false;         // FASTNN_B200_WIDE=0: CTA pairs keep 256-wide tiles
  bool conv_no_slab = false;    // FASTNN_B200_CONV_SLAB=0: the convolution gathers from global memory only
  int pace = 7;                 // FASTNN_B200_PACE=<0..8>: eighths of a tile's time its gather stores are spread over
};
const Tunables& tunables() {
  static const Tunables t = [] {
    Tunables v;
    auto num = [](const char* name, int fallback) {
      const char* e = std::getenv(name);
      return e != nullptr ? std::atoi(e) : fallback;
    };
    v.no_chunked = std::getenv("FASTNN_B200_NO_CHUNKED") != nullptr;
    v.cluster_k_off = num("FASTNN_B200_CLUSTER_K", 1) == 0;
    v.pdl = num("FASTNN_B200_PDL", 1) != 0;
    v.kb_per_stage = num("FASTNN_B200_KB_PER_STAGE", 0);
    v.stages = num("FASTNN_B200_STAGES", 0);
    v.group_m = num("FASTNN_B200_GROUP_M", 0);
    v.l2 = num("FASTNN_B200_L2", -1);
    v.no_wide = num("FASTNN_B200_WIDE", 1) == 0;
    v.conv_no_slab = num("FASTNN_B200_CONV_SLAB", 1) == 0;
    v.pace = num("FASTNN_B200_PACE", 7);
    if (v.pace < 0 || v.pace > 8) v.pace = 7;
    return v;
  }();
  return t;
}

struct LastCall {
  int path = 0, block_n = 0, split_k = 0, num_ctas = 0;
};
thread_local LastCall t_last;

#define FNN_CUDA_OK(call)                      \
  do {                                         \
    if ((call) != cudaSuccess) {               \
      (void)cudaGetLastError();                \
      return -1;                               \
    }                                          \
  } while (0)

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

DeviceState* current_state() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    (void)cudaGetLastError();
    return nullptr;
  }
  DeviceState* st = &g_dev[dev];
  return st->ready.load(std::memory_order_acquire) ? st : nullptr;
}

// The stream's scratch buffer of one of the two tables, grown when too small.  Growth is
// stream-ordered (cudaFreeAsync / cudaMallocAsync on the call's stream): kernels already queued on
// the stream keep their buffer until they have run, and nothing synchronises the device.  A
// stream under capture cannot grow its buffer (the allocation would belong to the graph): make
// the same call once before capturing.
int workspace_reserve(DeviceState* st, std::map<cudaStream_t, Workspace>& table, cudaStream_t s,
                      size_t need, float** out) {
  std::lock_guard<std::mutex> lock(st->ws_mutex);
  Workspace& ws = table[s];
  if (ws.bytes < need) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cap) != cudaSuccess) { (void)cudaGetLastError(); return -1; }
    if (cap != cudaStreamCaptureStatusNone) {
      std::fprintf(stderr, "fastnn_b200: a scratch buffer of %zu bytes is needed while the stream is "
                           "being captured; run the call once before the capture\n", need);
      return -1;
    }
    if (ws.ptr != nullptr) FNN_CUDA_OK(cudaFreeAsync(ws.ptr, s));
    ws.ptr = nullptr; ws.bytes = 0;
    void* ptr = nullptr;
    FNN_CUDA_OK(cudaMallocAsync(&ptr, need, s));
    ws.ptr = static_cast<float*>(ptr);
    ws.bytes = need;
  }
  *out = ws.ptr;
  return 0;
}

// Encoded tensor maps are a pure function of their arguments, and a training loop presents the
// same buffers with the same shapes over and over: a small direct-mapped cache in front of
// cuTensorMapEncodeTiled (three to five encodings per GEMM call otherwise).
struct MapKey {
  const void* base;
  uint64_t d[4], s[3];
  uint32_t box[3], kind;     // kind: 0 = 3-D 16-byte atoms, 1 = 3-D 32-byte atoms, 2 = 4-D 32-byte atoms
  bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapSlot {
  bool valid = false;
  MapKey key;
  CUtensorMap map;
};
constexpr int kMapCacheSlots = 512;
MapSlot g_map_cache[kMapCacheSlots];
std::mutex g_map_mutex;

inline size_t map_hash(const MapKey& k) {
  uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
  for (int i = 0; i < 4; ++i) h = (h ^ k.d[i]) * 0x100000001B3ull;
  for (int i = 0; i < 3; ++i) h = (h ^ k.s[i]) * 0x100000001B3ull;
  for (int i = 0; i < 3; ++i) h = (h ^ k.box[i]) * 0x100000001B3ull;
  h = (h ^ k.kind) * 0x100000001B3ull;
  return static_cast<size_t>(h >> 20) % kMapCacheSlots;
}
inline bool map_cache_get(const MapKey& k, CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  const MapSlot& s = g_map_cache[map_hash(k)];
  if (!s.valid || !(s.key == k)) return false;
  *out = s.map;
  return true;
}
inline void map_cache_put(const MapKey& k, const CUtensorMap& m) {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  MapSlot& s = g_map_cache[map_hash(k)];
  s.valid = true;
  s.key = k;
  s.map = m;
}

// 3-D FP32 tensor map, 128-byte swizzle span, zero fill outside the tensor.  `atom32` selects
// the 32-byte swizzle unit that MN-major TF32 operands need; otherwise the unit is 16 bytes.
bool encode_map(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1,
                bool atom32 = false) {
  const EncodeTiledFn encode = g_encode.load(std::memory_order_acquire);
  if (encode == nullptr) return false;
  MapKey key;
  std::memset(&key, 0, sizeof(key));          // padding bytes too: the key is compared bytewise
  key.base = base;
  key.d[0] = d0; key.d[1] = d1; key.d[2] = d2;
  key.s[0] = stride1_bytes; key.s[1] = stride2_bytes;
  key.box[0] = box0; key.box[1] = box1; key.box[2] = 1;
  key.kind = atom32 ? 1u : 0u;
  if (map_cache_get(key, map)) return true;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) map_cache_put(key, *map);
  return r == CUDA_SUCCESS;
}

// 4-D FP32 tensor map with the 32-byte-atom swizzle: the chunked view of an MN-major operand.
// Strides need not ascend: dimension 1 (k) strides by a whole row, dimension 2 (chunk) by 128 B.
bool encode_map4(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                 uint64_t d3, uint64_t stride1_bytes, uint64_t stride2_bytes,
                 uint64_t stride3_bytes, uint32_t box0, uint32_t box1, uint32_t box2) {
  const EncodeTiledFn encode = g_encode.load(std::memory_order_acquire);
  if (encode == nullptr) return false;
  MapKey key;
  std::memset(&key, 0, sizeof(key));
  key.base = base;
  key.d[0] = d0; key.d[1] = d1; key.d[2] = d2; key.d[3] = d3;
  key.s[0] = stride1_bytes; key.s[1] = stride2_bytes; key.s[2] = stride3_bytes;
  key.box[0] = box0; key.box[1] = box1; key.box[2] = box2;
  key.kind = 2u;
  if (map_cache_get(key, map)) return true;
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {stride1_bytes, stride2_bytes, stride3_bytes};
  cuuint32_t box[4] = {box0, box1, box2, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) map_cache_put(key, *map);
  return r == CUDA_SUCCESS;
}

struct Plan {
  int block_n, split_k, stages;
  bool pair;                        // 256 x block_n tiles on CTA pairs (cta_group::2)
  bool cluster_k = false;           // the K slices of a tile are the CTAs of one cluster
};

inline int log2_exact(int v) {      // 1 -> 0, 2 -> 1, 4 -> 2, 8 -> 3, 16 -> 4, anything else -1
  for (int i = 0; i <= 4; ++i)
    if (v == (1 << i)) return i;
  return -1;
}

int stages_for(int block_n, bool pair, int kb_per_stage);

// Pipeline stages of a cluster split-K CTA: one per k-block of its slice (at least two, at most
// what fits), and never a ring smaller than the partial tile that is written over it.
int ck_stages(int block_n, int kb_per_slice) {
  const size_t stage_b = fnn::kStageABytes + static_cast<size_t>(block_n) * fnn::kBlockK * 4;
  const size_t partial = static_cast<size_t>(fnn::kBlockM) * fnn::cluster_partial_pitch(block_n);
  const int for_partial = static_cast<int>((partial + stage_b - 1) / stage_b);
  int stages = kb_per_slice < 2 ? 2 : kb_per_slice;
  const int cap = stages_for(block_n, false, 1);
  if (stages > cap) stages = cap;
  if (stages < for_partial) stages = for_partial;      // for_partial <= cap for every block_n
  return stages;
}

// Co-resident CTAs of that kernel for cluster size 2^lg: CTAs small enough share an SM in pairs.
int ck_slots_for(const int* full, const int* half, int lg, int block_n, int kb_per_slice) {
  int slots = full[lg];
  if (half != nullptr && half[lg] > slots &&
      fnn::gemm_clusterk_smem_bytes(block_n, ck_stages(block_n, kb_per_slice)) <= kCkHalfSmem)
    slots = half[lg];
  return slots;
}

// Cycle model used to pick the tile shape and the K split.  Per 32-deep k-block (four MMAs) a
// CTA is bound either by the tensor pipe (block_n / 2 cycles at 4096 dense TF32 flop/clk/SM) or by
// reading its A and B stage from shared memory at 128 B/clk, or by the producer's TMA issue rate
// when an MN-major operand has to be fetched one 32-wide chunk per instruction (a_mn / b_mn:
// extent not a multiple of 32, so the single-box chunked view does not apply).  A CTA pair
// computes 256 x block_n with each CTA reading only half of B.
Plan choose_plan(int m, int n, int k, int batch, int num_sms, int max_clusters, bool a_mn,
                 bool b_mn, int pair_mode /* 0 auto, 1 never, 2 always */,
                 const int* ck_slots = nullptr /* DeviceState::ck_slots, or null: no cluster split-K */,
                 const int* ck_slots_half = nullptr) {
  const int num_kb = ceil_div(k, fnn::kBlockK);
  const int n32 = ceil_div(n, 32) * 32;
  const double out_bytes = 4.0 * m * n * batch;
  const double hbm_per_clk = 3400.0;     // 6.5 TB/s at 1.9 GHz
  const double in_bytes = 4.0 * batch * (1.0 * m * k + 1.0 * k * n);
  Plan best{32, 1, 4, false};
  double best_cost = 1e300;
  static const int splits[] = {1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64};
  for (int pair = 0; pair < 2; ++pair) {
    if (pair == 1 && (pair_mode == 1 || max_clusters < 1)) continue;
    if (pair == 0 && pair_mode == 2) continue;
    if (pair == 1 && pair_mode == 0 && m <= fnn::kBlockM) continue;
    const int tile_m = pair ? 2 * fnn::kBlockM : fnn::kBlockM;
    const int tiles_m = ceil_div(m, tile_m);
    const int slots = pair ? max_clusters : num_sms;
    for (int bn = pair ? 64 : 32; bn <= fnn::kMaxBlockN; bn += pair ? 64 : 32) {
      if (bn > n32 && bn > (pair ? 64 : 32)) break;
      const int tiles_n = ceil_div(n, bn);
      // skip widths whose last tile is mostly padding (more than 1/8 of the columns wasted)
      if ((tiles_n * bn - n32) * 8 > n32 && bn > (pair ? 64 : 32)) continue;
      const double a_bytes = 4096.0;
      const double b_bytes = (pair ? 16.0 : 32.0) * bn;
      const double t_smem = (a_bytes + b_bytes) / 128.0;
      // an operand fetched as one box per 32-wide chunk costs the producer ~90 cycles per box
      const double t_issue = 90.0 * ((a_mn ? 4 : 1) + (b_mn ? (pair ? bn / 64 : bn / 32) : 1));
      double t_kb = bn / 2.0 > t_smem ? bn / 2.0 : t_smem;
      if (t_issue > t_kb) t_kb = t_issue;
      // measured floor of one stage hand-over (wait, four MMAs, commit) in the issuing thread
      if (t_kb < 550.0) t_kb = 550.0;
      for (int s : splits) {
        if (s > 1 && num_kb / s < 2) break;
        const int kbps = ceil_div(num_kb, s);
        const int real_split = ceil_div(num_kb, kbps);
        const long long units = 1ll * batch * tiles_m * tiles_n * real_split;
        const double waves = static_cast<double>((units + slots - 1) / slots);
        // measured with hinted operand loads: a CTA pair with 256-wide tiles and two k-blocks per
        // stage is 3-5 % faster than single CTAs in a burst (4096^3, 8192^3) and 1-3 % faster over
        // 0.3 s and longer runs of 8192^3; on 32768 x 16384 x 4096 and its two gradient GEMMs under
        // the power cap the two are within +-4 % of each other, the sign changing from box to box.
        // Its per-tile hand-over between the two CTAs costs more and its per-stage saving grows
        // with K, so deep many-wave problems (K >= 4096) take pairs, the rest single CTAs.
        const double t_kb_scale =
            !pair ? 1.0 : ((bn == 256 && kbps >= 128 && waves >= 4.0) ? 0.97
                                                                       : ((bn == 256 && kbps >= 8) ? 1.05 : 1.12));
        // HBM time is stretched by idle SMs: a wave that fills only part of the machine still
        // takes a full wave
        const double imbalance = waves * slots * (pair ? 2 : 1) / ((pair ? 2.0 : 1.0) * units);
        const double partial_bytes = real_split > 1 ? real_split * out_bytes : 0.0;
        const double l2_discount = partial_bytes < 48e6 ? (1.0 / 3.0) : 1.0;   // stays in L2
        const double main_bytes = in_bytes + (real_split > 1 ? partial_bytes * l2_discount : out_bytes);
        const double t_hbm = main_bytes / hbm_per_clk * imbalance;
        const double t_cmp = waves * kbps * t_kb * t_kb_scale;
        double cycles = (t_hbm > t_cmp ? t_hbm : t_cmp) + waves * 800.0;
        if (real_split > 1)
          cycles += (partial_bytes * l2_discount + out_bytes) / hbm_per_clk + 5000.0;
        // prefer wider tiles, fewer splits and single CTAs on ties
        cycles *= 1.0 + 1e-4 * (8 - bn / 32) + 1e-3 * (real_split - 1) + 1e-4 * pair;
        if (cycles < best_cost) {
          best_cost = cycles;
          best.block_n = bn;
          best.split_k = real_split;
          best.pair = pair != 0;
          best.cluster_k = false;
        }
      }
      // The same K splits with the slices of a tile as one cluster (single CTAs, portable cluster
      // sizes): no partial tiles in global memory and no reduce launch; instead each CTA drains
      // its accumulator to shared memory and reads 512 * bn bytes from its cluster peers.
      for (int lg = 1; lg <= 4 && pair == 0 && ck_slots != nullptr; ++lg) {
        const int sk = 1 << lg;
        if (num_kb < 2 * sk) continue;
        // a short slice needs few stages: such CTAs fit two to an SM
        const int slots_ck = ck_slots_for(ck_slots, ck_slots_half, lg, bn, ceil_div(num_kb, sk));
        if (slots_ck < sk) continue;
        const long long units = 1ll * batch * tiles_m * tiles_n * sk;
        const double waves = static_cast<double>((units + slots_ck - 1) / slots_ck);
        const double imbalance = waves * slots_ck / units;
        const double t_hbm = (in_bytes + out_bytes) / hbm_per_clk * imbalance;
        const double t_cmp = waves * ceil_div(num_kb, sk) * t_kb;
        // measured on 512 x 256 x 784: two cluster barriers, the drain to shared memory and the
        // peer reads cost more the larger the cluster (its CTAs start and finish further apart)
        double cycles = (t_hbm > t_cmp ? t_hbm : t_cmp) + waves * (800.0 + 1500.0 + 300.0 * sk + 8.0 * bn);
        cycles *= 1.0 + 1e-4 * (8 - bn / 32) + 1e-3 * (sk - 1);
        if (cycles < best_cost) {
          best_cost = cycles;
          best.block_n = bn;
          best.split_k = sk;
          best.pair = false;
          best.cluster_k = true;
        }
      }
    }
  }
  return best;
}

// Deep products with at least a machine-full of tiles: the kind of tile is chosen by waves.
//   single CTAs, 128 x 256 tiles   one SM ingests 96 B/clk from L2 at full tensor rate (it can take 64)
//   CTA pairs,   256 x 256 tiles   64 B/clk per SM
//   CTA pairs,   256 x 512 tiles   48 B/clk per SM: two MMA groups share the A stage; the 512
//                                  accumulator columns are all of tensor memory, so the epilogue of a
//                                  tile no longer overlaps the next main loop
// Time = waves x (tile area per CTA) / rate, with the rates measured on 1024 x 8192 x 8192 (a burst:
// 630 / 681 / 732 TFLOP/s at 86 % tile-slot use, i.e. 1 : 1.08 : 1.16); the same figures rank
// 2048, 4096 and 8192 rows and 32768 x 16384 x 4096 with its gradient products the way they
// measured (8192^3: +7 % for the wide tile; K = 16384-32768: +10-18 %).  No K split: with this
// many tiles the partial sums cost more than the idle slots they would fill.  The fused bias +
// erf-GELU forward at K = 4096 lost 10 % on wide tiles (its epilogue is a fifth of a tile's time
// once nothing overlaps it), so a call with epilogue work takes them only for very deep K.
void refine_large_plan(Plan* plan, int m, int n, int k, int batch, int num_sms, int max_clusters,
                       bool a_mn, bool b_mn, int pair_mode, bool epilogue_work, bool allow_wide) {
  if (k < 2048 || a_mn || b_mn) return;       // per-chunk operand boxes are producer-bound: keep the model
  const long long t_single = 1ll * batch * ceil_div(m, fnn::kBlockM) * ceil_div(n, fnn::kMaxBlockN);
  if (t_single < num_sms) return;             // skinny outputs: the cost model's K split stands
  const bool pair_ok = pair_mode != 1 && max_clusters >= 1 && m > fnn::kBlockM;
  const long long t_pair = 1ll * batch * ceil_div(m, fnn::kPairBlockM) * ceil_div(n, fnn::kMaxBlockN);
  const long long t_wide = 1ll * batch * ceil_div(m, fnn::kPairBlockM) * ceil_div(n, fnn::kPairWideBlockN);
  auto waves = [](long long units, long long slots) { return static_cast<double>((units + slots - 1) / slots); };
  double best = pair_mode == 2 ? 1e300 : waves(t_single, num_sms);
  int kind = 0;                               // 0 single, 1 pair, 2 wide pair
  if (pair_ok) {
    const double c = waves(t_pair, max_clusters) / 1.08;
    if (c < best) { best = c; kind = 1; }
    if (allow_wide && n >= fnn::kPairWideBlockN && k >= (epilogue_work ? 16384 : 4096)) {
      const double cw = waves(t_wide, max_clusters) * 2.0 / 1.16;
      if (cw < best) { best = cw; kind = 2; }
    }
  }
  plan->split_k = 1;
  plan->cluster_k = false;
  plan->pair = kind != 0;
  if (kind == 1) plan->block_n = fnn::kMaxBlockN;
  if (kind == 2) plan->block_n = fnn::kPairWideBlockN;
  if (kind == 0 && plan->block_n > fnn::kMaxBlockN) plan->block_n = fnn::kMaxBlockN;
}

// choose_plan walks ~250 candidates (2-3 microseconds of host time, as much as the launch itself
// for a small GEMM), and training loops repeat a handful of shapes: remember the answers.  The
// slot tables are per device and constant after init, so the device's state pointer stands for
// them in the key.
Plan choose_plan_cached(const void* device_key, int m, int n, int k, int batch, int num_sms,
                        int max_clusters, bool a_mn, bool b_mn, int pair_mode, const int* ck_slots,
                        const int* ck_slots_half) {
  struct Key {
    const void* dev;
    int m, n, k, batch, flags;
    bool operator<(const Key& o) const {
      if (dev != o.dev) return dev < o.dev;
      if (m != o.m) return m < o.m;
      if (n != o.n) return n < o.n;
      if (k != o.k) return k < o.k;
      if (batch != o.batch) return batch < o.batch;
      return flags < o.flags;
    }
  };
  static std::map<Key, Plan> memo;
  static std::mutex memo_mutex;
  std::lock_guard<std::mutex> lock(memo_mutex);
  const Key key{device_key, m, n, k, batch,
                (a_mn ? 1 : 0) | (b_mn ? 2 : 0) | (pair_mode << 2) | (ck_slots != nullptr ? 16 : 0)};
  auto it = memo.find(key);
  if (it != memo.end()) return it->second;
  const Plan plan = choose_plan(m, n, k, batch, num_sms, max_clusters, a_mn, b_mn, pair_mode, ck_slots,
                                ck_slots_half);
  if (memo.size() >= 4096) memo.clear();
  memo.emplace(key, plan);
  return plan;
}

int stages_for(int block_n) { return stages_for(block_n, false, 1); }
int stages_for(int block_n, bool pair, int kb_per_stage) {
  const size_t stage = kb_per_stage * (fnn::kStageABytes + static_cast<size_t>(pair ? block_n / 2 : block_n) *
                                                               fnn::kBlockK * 4);
  const size_t avail = kMaxDynSmem - 1024 - fnn::kStagingBytes - fnn::kBarrierBytes;
  int s = static_cast<int>(avail / stage);
  if (s > fnn::kMaxStages) s = fnn::kMaxStages;
  return s;
}

struct GemmArgs {
  int layout;
  const float *a, *b;
  float* c;
  int m, n, k, batch;
  long long lda, ldb, ldc, sa, sb, sc;
  float alpha, beta;
  const float* bias;
  int act;
  cudaStream_t stream;
  // backward epilogue (act 3 / 4): saved pre-activations and the optional column-sum output
  const float* aux = nullptr;
  long long ld_aux = 0;
  float* colsum = nullptr;
  // second operand pair of C = A.B + A2.B2 (same layout, m, n; batch 1) and a second bias
  const float *a2 = nullptr, *b2 = nullptr;
  int k2 = 0;
  long long lda2 = 0, ldb2 = 0;
  const float* bias2 = nullptr;
  int force_split_k = 0;     // > 0: overrides the planner's K split (callers that own the workspace)
  // gather: the location of C's rows in up to kMaxPeers other GPUs' memory (peer-mapped pointers);
  // every finished tile is stored there as well as to c
  float* const* peer_c = nullptr;
  int n_peers = 0;
  // or, instead of the peers: the NVLink multicast address of those rows (one multimem.st per
  // 16 bytes reaches every GPU's C, this one's included; c itself is then not written directly)
  float* mc_c = nullptr;
};

bool tma_operands_ok(const GemmArgs& g) {
  if (g.k < 1) return false;
  if (!aligned16(g.a) || !aligned16(g.b)) return false;
  if ((g.lda & 3) || (g.ldb & 3)) return false;
  if (g.batch > 1 && ((g.sa & 3) || (g.sb & 3))) return false;
  // tensor-map limits: strides below 2^40 bytes
  const long long lim = (1ll << 40) / 4;
  if (g.lda >= lim || g.ldb >= lim || g.sa >= lim || g.sb >= lim) return false;
  return true;
}

int launch_simt(const GemmArgs& g) {
  fnn::SimtParams p;
  p.a = g.a; p.b = g.b; p.c = g.c; p.bias = g.bias;
  p.m = g.m; p.n = g.n; p.k = g.k; p.batch = g.batch;
  p.a_bs = g.sa; p.b_bs = g.sb; p.c_bs = g.sc; p.ldc = g.ldc;
  if (g.layout == FASTNN_B200_TN) { p.a_rs = 1; p.a_cs = g.lda; } else { p.a_rs = g.lda; p.a_cs = 1; }
  if (g.layout == FASTNN_B200_NT) { p.b_rs = 1; p.b_cs = g.ldb; } else { p.b_rs = g.ldb; p.b_cs = 1; }
  p.alpha = g.alpha; p.beta = g.beta; p.act = g.act > 2 ? 0 : g.act;
  const int gx = ceil_div(g.n, fnn::kSimtTile), gy = ceil_div(g.m, fnn::kSimtTile);
  if (gy > 65535) return -1;
  for (int b0 = 0; b0 < g.batch; b0 += 65535) {
    fnn::SimtParams q = p;
    q.a += b0 * p.a_bs; q.b += b0 * p.b_bs; q.c += b0 * p.c_bs;
    const int nb = g.batch - b0 < 65535 ? g.batch - b0 : 65535;
    fnn::gemm_simt_kernel<<<dim3(gx, gy, nb), 256, 0, g.stream>>>(q);
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  FNN_CUDA_OK(cudaGetLastError());
  // backward epilogue as two small passes (only batch 1 reaches here with aux / colsum set)
  if (g.act > 2 && g.aux != nullptr) {
    long long blocks = (1ll * g.m * g.n + 255) / 256;
    if (blocks > 4096) blocks = 4096;
    fnn::act_grad_inplace_kernel<<<static_cast<unsigned>(blocks), 256, 0, g.stream>>>(
        g.c, g.aux, g.m, g.n, g.ldc, g.ld_aux, g.act);
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  if (g.colsum != nullptr) {
    fnn::colsum_kernel<<<ceil_div(g.n, 256), 256, 0, g.stream>>>(g.c, g.colsum, g.m, g.n, g.ldc);
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  FNN_CUDA_OK(cudaGetLastError());
  t_last = LastCall{1, 0, 1, gx * gy * g.batch};
  return 0;
}

int launch_tcgen05(DeviceState* st, const GemmArgs& g, const Policy& pol) {
  const Tunables& tune = tunables();
  const bool no_chunk = tune.no_chunked;
  const bool a_mn = (g.layout == FASTNN_B200_TN) && ((g.m % 32) != 0 || no_chunk);
  const bool b_mn = (g.layout != FASTNN_B200_NT) && ((g.n % 32) != 0 || no_chunk);
  const bool dual = g.a2 != nullptr;       // C = A.B + A2.B2: single-CTA kernel, one K range
  const bool gather = g.n_peers > 0 || g.mc_c != nullptr;   // tiles also go to other GPUs: whole K per tile
  const int pair_mode = dual ? 1 : ((pol.policy == 3 || pol.policy >= 5) ? 1 : (pol.policy == 4 ? 2 : 0));
  // the backward epilogue is not linear in the partial sums, and the column sums use the workspace
  const bool backward = g.aux != nullptr || g.colsum != nullptr;
  // cluster split-K writes C itself: not for callers that want the raw partial tiles
  const bool ck_allowed = !backward && !gather && g.force_split_k == 0 && pol.policy != 6 &&
                          pol.policy != 3 && pol.policy != 4 && !tune.cluster_k_off;
  Plan plan = choose_plan_cached(st, g.m, g.n, g.k + (dual ? g.k2 : 0), g.batch, st->num_sms,
                                 st->max_clusters, a_mn, b_mn, pair_mode,
                                 ck_allowed ? st->ck_slots : nullptr, st->ck_slots_half);
  if (!dual && !gather)
    refine_large_plan(&plan, g.m, g.n, g.k, g.batch, st->num_sms, st->max_clusters, a_mn, b_mn, pair_mode,
                      g.bias != nullptr || g.act != 0 || backward, !tune.no_wide);
  else if (gather && !dual) {
    // Tiles leave for the peers as they finish, so a K split is out, and when the links rather than
    // the tensor cores bound the launch (peer bytes at ~0.7 TB/s against the product at ~0.7
    // PFLOP/s) what counts is how soon the first tiles are done and how evenly the rest follow:
    // single-CTA 128 x 256 tiles finish in half the time of a CTA pair's tile and come in twice as
    // many waves, so the stores of one wave overlap the main loops of the next.
    const double t_link = 4.0 * g.m * g.n * g.batch * (g.mc_c != nullptr ? 1 : g.n_peers) / 0.7e12;
    const double t_math = 2.0 * g.m * g.n * g.batch * static_cast<double>(g.k) / 0.7e15;
    const int mode = (t_link > 0.6 * t_math && pair_mode == 0) ? 1 : pair_mode;
    refine_large_plan(&plan, g.m, g.n, g.k, g.batch, st->num_sms, st->max_clusters, a_mn, b_mn, mode,
                      g.bias != nullptr || g.act != 0, !tune.no_wide);
    if (mode == 1 && pair_mode == 0) plan.pair = false;
  }
  if (pol.block_n > 0) plan.block_n = pol.block_n;
  if (!plan.pair && plan.block_n > fnn::kMaxBlockN) plan.block_n = fnn::kMaxBlockN;
  if (pol.split_k > 0) { plan.split_k = pol.split_k; plan.cluster_k = false; }
  if (pol.policy == 5) plan.cluster_k = ck_allowed;            // forced: split_k is the cluster size
  if (backward || gather) { plan.split_k = 1; plan.cluster_k = false; }
  if (g.force_split_k > 0) plan.split_k = g.force_split_k;
  if (plan.pair && (plan.block_n % 64) != 0) plan.block_n = ceil_div(plan.block_n, 64) * 64;
  const int num_kb1 = ceil_div(g.k, fnn::kBlockK);
  const int num_kb = num_kb1 + (dual ? ceil_div(g.k2, fnn::kBlockK) : 0);
  if (plan.split_k > num_kb) plan.split_k = num_kb;
  if (plan.cluster_k) {
    // a cluster size the device can place, every slice at least one k-block, and a partial tile
    // that fits the stage ring it is written over; otherwise the workspace form of the same split
    const int lg = log2_exact(plan.split_k);
    if (plan.pair || lg < 1 || num_kb < plan.split_k ||
        ck_slots_for(st->ck_slots, st->ck_slots_half, lg, plan.block_n,
                     ceil_div(num_kb, plan.split_k)) < plan.split_k)
      plan.cluster_k = false;
  }
  const int kbps = ceil_div(num_kb, plan.split_k);
  if (!plan.cluster_k) plan.split_k = ceil_div(num_kb, kbps);
  // CTA pairs with wide tiles take two k-blocks per stage: the issuing thread's per-stage
  // cost (wait, commit, loop) is then paid once per eight MMAs instead of once per four
  int kb_per_stage = (plan.pair && plan.block_n == 256 && kbps >= 8) ? 2 : 1;
  if (plan.pair && tune.kb_per_stage >= 1 && tune.kb_per_stage <= 4) kb_per_stage = tune.kb_per_stage;
  if (plan.block_n > fnn::kMaxBlockN) kb_per_stage = 1;     // a wide stage already holds eight MMAs
  plan.stages = stages_for(plan.block_n, plan.pair, kb_per_stage);
  if (plan.stages < 2) { kb_per_stage = 1; plan.stages = stages_for(plan.block_n, plan.pair, 1); }
  if (tune.stages >= 1 && tune.stages < plan.stages) plan.stages = tune.stages;
  // A cluster split-K CTA lives for one K slice: no more stages than the slice has k-blocks (but
  // a ring that holds the partial tile), and one accumulator.  The smaller footprint lets CTAs of
  // consecutive launches, or of two clusters, share an SM.  TMEM allocation blocks until columns
  // are free, and a CTA waiting there while a cluster peer on the same SM waits for it at the
  // cluster barrier would never get them: the shared-memory request is kept large enough that the
  // CTAs that fit one SM never ask for more than the 512 columns together.
  int ck_tmem_cols = 0;
  size_t ck_smem = 0;
  if (plan.cluster_k) {
    plan.stages = ck_stages(plan.block_n, ceil_div(num_kb, plan.split_k));
    ck_tmem_cols = 32;
    while (ck_tmem_cols < plan.block_n) ck_tmem_cols *= 2;
    ck_smem = fnn::gemm_clusterk_smem_bytes(plan.block_n, plan.stages);
    const size_t sm_smem = 228 * 1024;                      // per SM, 1 KiB reserved per CTA
    const size_t ctas_ok = 512 / ck_tmem_cols;              // CTAs whose accumulators fit together
    const size_t floor_bytes = sm_smem / (ctas_ok + 1) + 1; // ctas_ok + 1 of these do not fit
    if (ck_smem < floor_bytes) ck_smem = floor_bytes;
  }

  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.m = g.m; p.n = g.n; p.k = g.k; p.batch = g.batch;
  p.block_n = plan.block_n;
  p.num_stages = plan.stages;
  p.tiles_m = ceil_div(g.m, plan.pair ? fnn::kPairBlockM : fnn::kBlockM);
  p.tiles_n = ceil_div(g.n, plan.block_n);
  p.num_kb = num_kb;
  p.num_kb1 = num_kb1;
  p.split_k = plan.split_k;
  p.kb_per_split = kbps;
  p.kb_per_stage = kb_per_stage;
  // two MMA groups (two issuing threads) for the wide pair tile, 512 = 2 x 256; a 256-wide tile as
  // 2 x 128 measured slower than one group (562-570 against 619-621 TFLOP/s on the fused forward)
  const int mma_groups = (plan.pair && plan.block_n > fnn::kMaxBlockN) ? 2 : 1;
  p.mma_groups = mma_groups;
  const long long units = 1ll * g.batch * p.tiles_m * p.tiles_n * plan.split_k;
  if (units > 0x7fffffffll) return -1;
  p.total_units = static_cast<int>(units);
  p.a_mn_major = (g.layout == FASTNN_B200_TN) ? 1 : 0;
  p.b_mn_major = (g.layout == FASTNN_B200_NT) ? 0 : 1;
  p.alpha = g.alpha; p.beta = g.beta; p.bias = g.bias; p.bias2 = g.bias2; p.act = g.act;
  p.status = st->status;
  p.spin_budget = st->spin_budget;
  p.group_m = plan.pair ? fnn::kGroupM / 2 : fnn::kGroupM;     // 2048 rows of C either way
  // Operand loads carry the evict-unchanged L2 policy.  A load with the default policy also
  // demotes the line it hits, a second tag operation per sector: with the hint the L2 answers the
  // same 24x-operand-bytes of tile reads with half the lookups (ncu at 4096^3: lts__throughput
  // 61 % -> 34 %, cross-partition requests 15.3 M -> 4.5 M, DRAM bytes unchanged).  Measured at
  // 8192^3 on single CTAs: +10 % in a burst, +19 % sustained under the power cap.
  p.l2_a = 3; p.l2_b = 3; p.l2_c = 0;
  if (tune.group_m >= 1 && tune.group_m <= 1024) p.group_m = tune.group_m;
  if (tune.l2 >= 0) {                                           // digits: C, A, B policy
    const int v = tune.l2;
    p.l2_c = (v / 100) % 10 % 5; p.l2_a = (v / 10) % 10 % 5; p.l2_b = v % 10 % 5;
  }

  // output target: C itself, or the split-K workspace
  float* out = g.c;
  long long out_ld = g.ldc, out_bs = g.sc;
  long long out_z = g.batch;
  p.cluster_k = plan.cluster_k ? 1 : 0;
  p.n_peers = g.n_peers;
  p.mc_c = g.mc_c;
  p.tmem_cols = ck_tmem_cols;
  p.cluster_vec = (plan.cluster_k && (g.n & 3) == 0 && aligned16(g.c) && (g.ldc & 3) == 0 &&
                   (g.batch == 1 || (g.sc & 3) == 0)) ? 1 : 0;
  if (plan.split_k > 1 && !plan.cluster_k) {
    const size_t need = sizeof(float) * static_cast<size_t>(g.m) * g.n * g.batch * plan.split_k;
    if (workspace_reserve(st, st->workspaces, g.stream, need, &out) != 0) return -1;
    out_ld = g.n;
    out_bs = static_cast<long long>(g.m) * g.n;
    out_z = static_cast<long long>(g.batch) * plan.split_k;
    p.bias = nullptr;
  }
  p.aux = g.aux; p.ld_aux = g.ld_aux;
  const int slabs = ceil_div(g.m, 32);              // 32-row slabs of C, one partial row each
  if (g.colsum != nullptr) {
    const size_t need = sizeof(float) * static_cast<size_t>(slabs) * g.n;
    if (workspace_reserve(st, st->workspaces, g.stream, need, &p.colsum) != 0) return -1;
  }
  const bool tma_store = !plan.cluster_k && aligned16(out) && (out_ld & 3) == 0 && (out_z == 1 || (out_bs & 3) == 0) &&
                         (plan.split_k > 1 || g.beta == 0.0f) && out_ld < (1ll << 38) &&
                         out_bs < (1ll << 38);
  p.store_mode = tma_store ? 0 : 1;
  p.c = out; p.ldc = out_ld; p.c_batch_stride = out_bs;
  if (gather && !tma_store) return -1;        // peer tiles leave by TMA store only

  CUtensorMap tmA, tmB, tmC;
  const uint64_t B = static_cast<uint64_t>(g.batch);
  const uint64_t sa_bytes = (g.batch > 1 ? g.sa : g.lda * (p.a_mn_major ? g.k : g.m)) * 4ull;
  const uint64_t sb_bytes = (g.batch > 1 ? g.sb : g.ldb * (p.b_mn_major ? g.k : g.n)) * 4ull;
  bool ok;
  // An MN-major operand whose contiguous extent is a multiple of 32 is also addressable as
  // (32, k, extent/32, batch): one box then brings all 32-wide chunks of a stage, laid out
  // chunk-major in shared memory exactly as the per-chunk boxes would.
  p.a_chunked = (p.a_mn_major && (g.m % 32) == 0 && !no_chunk) ? 1 : 0;
  p.b_chunked = (p.b_mn_major && (g.n % 32) == 0 && !no_chunk) ? 1 : 0;
  if (!p.a_mn_major)
    ok = encode_map(&tmA, g.a, g.k, g.m, B, g.lda * 4ull, sa_bytes, fnn::kBlockK, fnn::kBlockM);
  else {
    ok = false;
    if (p.a_chunked)
      ok = encode_map4(&tmA, g.a, 32, g.k, g.m / 32, B, g.lda * 4ull, 128ull, sa_bytes, 32,
                       fnn::kBlockK, fnn::kBlockM / 32);
    if (!ok) {   // driver refused the chunked view (or it does not apply): one box per chunk
      p.a_chunked = 0;
      ok = encode_map(&tmA, g.a, g.m, g.k, B, g.lda * 4ull, sa_bytes, 32, fnn::kBlockK, true);
    }
  }
  // B columns one load brings: a CTA's half of one MMA group (a wide tile is two groups of 256)
  const int b_cols = plan.pair ? (plan.block_n / mma_groups) / 2
                               : plan.block_n;
  if (!p.b_mn_major)
    ok = ok && encode_map(&tmB, g.b, g.k, g.n, B, g.ldb * 4ull, sb_bytes, fnn::kBlockK, b_cols);
  else {
    bool okb = false;
    if (p.b_chunked)
      okb = encode_map4(&tmB, g.b, 32, g.k, g.n / 32, B, g.ldb * 4ull, 128ull, sb_bytes, 32,
                        fnn::kBlockK, b_cols / 32);
    if (!okb) {
      p.b_chunked = 0;
      okb = encode_map(&tmB, g.b, g.n, g.k, B, g.ldb * 4ull, sb_bytes, 32, fnn::kBlockK, true);
    }
    ok = ok && okb;
  }
  if (tma_store) {
    const uint64_t sc_bytes = (out_z > 1 ? out_bs : out_ld * g.m) * 4ull;
    ok = ok && encode_map(&tmC, out, g.n, g.m, static_cast<uint64_t>(out_z), out_ld * 4ull,
                          sc_bytes, 32, 32);
  } else {
    std::memset(&tmC, 0, sizeof(tmC));
  }
  CUtensorMap tmA2 = tmA, tmB2 = tmB;
  if (dual) {                                    // NT only: both operands of both pairs K-major
    ok = ok && encode_map(&tmA2, g.a2, g.k2, g.m, 1, g.lda2 * 4ull, g.lda2 * 4ull * g.m,
                          fnn::kBlockK, fnn::kBlockM);
    ok = ok && encode_map(&tmB2, g.b2, g.k2, g.n, 1, g.ldb2 * 4ull, g.ldb2 * 4ull * g.n,
                          fnn::kBlockK, b_cols);
  }
  fnn::PeerMaps peers;
  if (gather) std::memset(&peers, 0, sizeof(peers));
  if (g.n_peers > 0) {
    // the same rows of C on the other GPUs: identical shape and strides, another base address
    const uint64_t sc_bytes = (out_z > 1 ? out_bs : out_ld * g.m) * 4ull;
    for (int i = 0; i < g.n_peers && ok; ++i)
      ok = g.peer_c[i] != nullptr && aligned16(g.peer_c[i]) &&
           encode_map(&peers.m[i], g.peer_c[i], g.n, g.m, static_cast<uint64_t>(out_z), out_ld * 4ull,
                      sc_bytes, 32, 32);
  }
  if (gather) p.pace_gather = tune.pace;
  if (!ok) return -1;

  int grid;
  if (plan.pair) {
    const int clusters = p.total_units < st->max_clusters ? p.total_units : st->max_clusters;
    grid = 2 * clusters;
    const size_t smem = fnn::gemm_pair_smem_bytes(plan.block_n, plan.stages, kb_per_stage);
    if (gather)
      fnn::gemm_tf32_pair_gather_kernel<<<grid, fnn::kNumThreadsPair, smem, g.stream>>>(tmA, tmB, tmC, peers, p);
    else
      fnn::gemm_tf32_pair_kernel<<<grid, fnn::kNumThreadsPair, smem, g.stream>>>(tmA, tmB, tmC, p);
  } else if (gather) {
    grid = p.total_units < st->num_sms ? p.total_units : st->num_sms;
    const size_t smem = fnn::gemm_smem_bytes(plan.block_n, plan.stages);
    const bool epilogue_work = g.act != 0 || g.bias != nullptr;
    fnn::gemm_tf32_gather_kernel<<<grid, epilogue_work ? fnn::kNumThreadsWide : fnn::kNumThreads, smem,
                                   g.stream>>>(tmA, tmB, tmC, peers, p);
  } else if (plan.cluster_k) {
    // one CTA per unit, the split_k slices of a tile as one cluster; also a programmatic dependent
    grid = p.total_units;
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(fnn::kNumThreadsWide, 1, 1);
    cfg.dynamicSmemBytes = ck_smem;
    cfg.stream = g.stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = static_cast<unsigned>(plan.split_k);
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 2;
    FNN_CUDA_OK(cudaLaunchKernelEx(&cfg, fnn::gemm_tf32_clusterk_kernel, tmA, tmB, tmC, tmA2, tmB2, p));
  } else {
    grid = p.total_units < st->num_sms ? p.total_units : st->num_sms;
    const size_t smem = fnn::gemm_smem_bytes(plan.block_n, plan.stages);
    // bias, activation, derivative and column sums are a second pass over every output element by
    // the epilogue warps alone: eight of them keep it under a short-K main loop
    const bool epilogue_work = g.act != 0 || g.bias != nullptr || g.colsum != nullptr;
    const int threads = (epilogue_work && plan.split_k == 1) ? fnn::kNumThreadsWide : fnn::kNumThreads;
    if (tune.pdl) {
      // programmatic dependent launch: this grid's CTAs may start on SMs the previous kernel of
      // the stream has left; the kernel waits for that kernel's completion before it touches
      // global memory (griddepcontrol.wait), so only its set-up overlaps
      cudaLaunchConfig_t cfg;
      std::memset(&cfg, 0, sizeof(cfg));
      cfg.gridDim = dim3(grid, 1, 1);
      cfg.blockDim = dim3(threads, 1, 1);
      cfg.dynamicSmemBytes = smem;
      cfg.stream = g.stream;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr.val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      FNN_CUDA_OK(cudaLaunchKernelEx(&cfg, fnn::gemm_tf32_kernel, tmA, tmB, tmC, tmA2, tmB2, p));
    } else {
      fnn::gemm_tf32_kernel<<<grid, threads, smem, g.stream>>>(tmA, tmB, tmC, tmA2, tmB2, p);
    }
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  FNN_CUDA_OK(cudaGetLastError());

  if (plan.split_k > 1 && !plan.cluster_k) {
    const long long total = 1ll * g.m * g.n * g.batch;
    const bool vec = (g.n & 3) == 0 && aligned16(g.c) && (g.ldc & 3) == 0 && (g.sc & 3) == 0 &&
                     (g.bias == nullptr || aligned16(g.bias)) &&
                     (g.bias2 == nullptr || aligned16(g.bias2));
    long long work = vec ? total / 4 : total;
    long long blocks = (work + 255) / 256;
    const long long cap = 8ll * st->num_sms;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    // also a programmatic dependent: its launch overlaps the GEMM's last tiles, and it waits for
    // the GEMM's completion (griddepcontrol.wait) before it reads a partial sum
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(static_cast<unsigned>(blocks), 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = g.stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const float* ws_f = out;
    if (vec)
      FNN_CUDA_OK(cudaLaunchKernelEx(&cfg, fnn::splitk_reduce_vec4_kernel,
                                     reinterpret_cast<const float4*>(ws_f), g.c, g.bias, g.m, g.n, g.batch,
                                     plan.split_k, g.ldc, g.sc, g.alpha, g.beta, g.act, g.bias2));
    else
      FNN_CUDA_OK(cudaLaunchKernelEx(&cfg, fnn::splitk_reduce_kernel, ws_f, g.c, g.bias, g.m, g.n,
                                     g.batch, plan.split_k, g.ldc, g.sc, g.alpha, g.beta, g.act, g.bias2));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    FNN_CUDA_OK(cudaGetLastError());
  }
  if (g.colsum != nullptr) {          // slab partials -> column sums, slabs added in order
    fnn::colsum_slabs_kernel<<<ceil_div(g.n, 32), 1024, 0, g.stream>>>(p.colsum, g.colsum, slabs, g.n);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    FNN_CUDA_OK(cudaGetLastError());
  }
  t_last = LastCall{plan.pair ? 3 : (plan.cluster_k ? 6 : 2), plan.block_n, plan.split_k, grid};
  return 0;
}

int gemm_dispatch(const GemmArgs& g);

// The gather for operands or outputs TMA cannot address (row lengths that are not multiples of
// four floats, unaligned bases): the ordinary GEMM into this GPU's C, then one strided copy per
// destination on the same stream.  Not overlapped with the product -- a correctness path for odd
// shapes; aligned shapes take the kernels whose epilogue stores to the peers tile by tile.
int gather_by_copies(const GemmArgs& g) {
  GemmArgs local = g;
  local.peer_c = nullptr;
  local.n_peers = 0;
  const int rc = gemm_dispatch(local);
  if (rc != 0) return rc;
  const bool dense_batches = g.batch == 1 || g.sc == 1ll * g.m * g.ldc;
  for (int i = 0; i < g.n_peers; ++i) {
    if (g.peer_c[i] == nullptr) return -1;
    if (dense_batches) {
      FNN_CUDA_OK(cudaMemcpy2DAsync(g.peer_c[i], sizeof(float) * g.ldc, g.c, sizeof(float) * g.ldc,
                                    sizeof(float) * g.n, static_cast<size_t>(g.m) * g.batch,
                                    cudaMemcpyDeviceToDevice, g.stream));
    } else {
      for (int b = 0; b < g.batch; ++b)
        FNN_CUDA_OK(cudaMemcpy2DAsync(g.peer_c[i] + b * g.sc, sizeof(float) * g.ldc, g.c + b * g.sc,
                                      sizeof(float) * g.ldc, sizeof(float) * g.n, g.m,
                                      cudaMemcpyDeviceToDevice, g.stream));
    }
  }
  return 0;
}

int gemm_dispatch(const GemmArgs& g) {
  if (g.layout < 0 || g.layout > 2) return -1;
  if (g.m < 0 || g.n < 0 || g.k < 0 || g.batch < 0) return -1;
  if (g.act < 0 || g.act > 4 || (g.act > 2 && g.aux == nullptr)) return -1;
  if (g.m == 0 || g.n == 0 || g.batch == 0) return 0;          // nothing to write
  if (g.c == nullptr || (g.k > 0 && (g.a == nullptr || g.b == nullptr))) return -1;
  // leading dimensions must cover a row
  const long long a_row = (g.layout == FASTNN_B200_TN) ? g.m : g.k;
  const long long b_row = (g.layout == FASTNN_B200_NT) ? g.k : g.n;
  if (g.lda < a_row || g.ldb < b_row || g.ldc < g.n) return -1;

  if (g.n_peers < 0 || g.n_peers > fnn::kMaxPeers || (g.n_peers > 0 && g.peer_c == nullptr)) return -1;
  DeviceState* st = current_state();
  if (st == nullptr) return -1;                                   // fastnn_cuda_init not called
  const Policy pol = t_policy;
  const bool can_tma = tma_operands_ok(g);
  if (g.n_peers > 0 || g.mc_c != nullptr) {
    bool stores_ok = can_tma && pol.policy != 1 && g.beta == 0.0f && aligned16(g.c) && (g.ldc & 3) == 0 &&
                     (g.batch == 1 || (g.sc & 3) == 0) && g.ldc < (1ll << 38) && g.sc < (1ll << 38);
    for (int i = 0; i < g.n_peers && stores_ok; ++i) stores_ok = g.peer_c[i] != nullptr && aligned16(g.peer_c[i]);
    if (g.mc_c != nullptr) {
      // 16-byte multicast stores of whole row segments; no other form exists for this destination
      if (g.n_peers > 0 || !stores_ok || !aligned16(g.mc_c) || (g.n & 3) != 0) return -1;
    } else if (!stores_ok) {
      return gather_by_copies(g);
    }
  }
  if (pol.policy >= 2 && !can_tma) return -1;
  if (pol.policy == 1 || !can_tma) return launch_simt(g);
  return launch_tcgen05(st, g, pol);
}

// C = A.B^T + A2.B2^T + bias + bias2 (NT, batch 1).  One launch with both K ranges in one
// accumulator when TMA can address all four operands, else two dependent launches.
int dual_dispatch(GemmArgs g) {
  const bool pair2_ok = g.k2 >= 1 && aligned16(g.a2) && aligned16(g.b2) && (g.lda2 & 3) == 0 &&
                        (g.ldb2 & 3) == 0;
  const bool fused = t_policy.policy != 1 && tma_operands_ok(g) && pair2_ok;
  if (fused) return gemm_dispatch(g);
  GemmArgs first = g;
  first.a2 = first.b2 = nullptr; first.k2 = 0; first.bias2 = nullptr;
  int rc = gemm_dispatch(first);
  if (rc != 0) return rc;
  GemmArgs second = first;
  second.a = g.a2; second.b = g.b2; second.k = g.k2; second.lda = g.lda2; second.ldb = g.ldb2;
  second.beta = 1.0f; second.bias = g.bias2;
  return gemm_dispatch(second);
}

// The driver's tensor-map encoder, looked up once per process.
int resolve_encoder() {
  if (g_encode.load(std::memory_order_acquire) != nullptr) return 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  FNN_CUDA_OK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
  if (qres != cudaDriverEntryPointSuccess || fn == nullptr) return -1;
  g_encode.store(reinterpret_cast<EncodeTiledFn>(fn), std::memory_order_release);
  return 0;
}

}  // namespace

// ============================================================ drop-in symbols ===

extern "C" int fastnn_cuda_init(int device_id) {
  if (device_id < 0 || device_id >= kMaxDevices) return -1;
  FNN_CUDA_OK(cudaSetDevice(device_id));
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState& st = g_dev[device_id];
  if (st.ready.load(std::memory_order_acquire)) return 0;
  cudaDeviceProp prop;
  FNN_CUDA_OK(cudaGetDeviceProperties(&prop, device_id));
  if (prop.major != 10) {
    std::fprintf(stderr, "fastnn_b200: device %d is sm_%d%d; this library carries sm_100a code only\n",
                 device_id, prop.major, prop.minor);
    return -1;
  }
  if (resolve_encoder() != 0) return -1;
  FNN_CUDA_OK(cudaFuncSetAttribute(fnn::gemm_tf32_kernel,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kMaxDynSmem)));
  FNN_CUDA_OK(cudaFuncSetAttribute(fnn::gemm_tf32_gather_kernel,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kMaxDynSmem)));
  FNN_CUDA_OK(cudaFuncSetAttribute(fnn::gemm_tf32_pair_gather_kernel,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kMaxDynSmem)));
  FNN_CUDA_OK(cudaFuncSetAttribute(fnn::conv2d_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kMaxDynSmem)));
  FNN_CUDA_OK(cudaFuncSetAttribute(fnn::conv2d_tf32_slab_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kMaxDynSmem)));
  FNN_CUDA_OK(cudaFuncSetAttribute(fnn::conv2d_tf32_slab_dual_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kMaxDynSmem)));
  FNN_CUDA_OK(cudaFuncSetAttribute(fnn::conv2d_wgrad_slab_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kMaxDynSmem)));
  FNN_CUDA_OK(cudaFuncSetAttribute(fnn::attention_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kMaxDynSmem)));
  FNN_CUDA_OK(cudaFuncSetAttribute(fnn::conv2d_wgrad_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kMaxDynSmem)));
  st.num_sms = prop.multiProcessorCount;
  FNN_CUDA_OK(cudaFuncSetAttribute(fnn::gemm_tf32_clusterk_kernel,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kMaxDynSmem)));
  // clusters of 16 are beyond the portable limit of 8; a device that refuses them reports no slots
  if (cudaFuncSetAttribute(fnn::gemm_tf32_clusterk_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed,
                           1) != cudaSuccess)
    (void)cudaGetLastError();
  for (int pass = 0; pass < 2; ++pass)
  for (int lg = 1; lg <= 4; ++lg) {
    // how many CTAs of the cluster split-K kernel fit at once at cluster size 2, 4, 8, 16 (a
    // cluster inside one GPC), with one CTA per SM and with two
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(((2 * prop.multiProcessorCount) >> lg) << lg, 1, 1);
    cfg.blockDim = dim3(fnn::kNumThreadsWide, 1, 1);
    cfg.dynamicSmemBytes = pass == 0 ? kMaxDynSmem : kCkHalfSmem;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 1u << lg; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, fnn::gemm_tf32_clusterk_kernel, &cfg) != cudaSuccess) {
      (void)cudaGetLastError();
      clusters = 0;
    }
    (pass == 0 ? st.ck_slots : st.ck_slots_half)[lg] = clusters << lg;
  }
  FNN_CUDA_OK(cudaFuncSetAttribute(fnn::gemm_tf32_pair_kernel,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kMaxDynSmem)));
  {
    // how many CTA pairs of the pair kernel can be resident at once (normally one per TPC)
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2 * prop.multiProcessorCount, 1, 1);
    cfg.blockDim = dim3(fnn::kNumThreadsPair, 1, 1);
    cfg.dynamicSmemBytes = fnn::gemm_pair_smem_bytes(fnn::kMaxBlockN, stages_for(fnn::kMaxBlockN, true, 1), 1);
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, fnn::gemm_tf32_pair_kernel, &cfg) != cudaSuccess) {
      (void)cudaGetLastError();
      clusters = 0;
    }
    st.max_clusters = clusters;
  }
  if (std::getenv("FASTNN_B200_VERBOSE") != nullptr)
    std::fprintf(stderr, "fastnn_b200: device %d: %d SMs, %d CTA pairs; cluster split-K CTAs resident at "
                 "cluster size 2/4/8/16: %d/%d/%d/%d (full footprint), %d/%d/%d/%d (half)\n",
                 device_id, prop.multiProcessorCount, st.max_clusters, st.ck_slots[1], st.ck_slots[2],
                 st.ck_slots[3], st.ck_slots[4], st.ck_slots_half[1], st.ck_slots_half[2],
                 st.ck_slots_half[3], st.ck_slots_half[4]);
  FNN_CUDA_OK(cudaMalloc(&st.status, sizeof(unsigned int)));
  FNN_CUDA_OK(cudaMemset(st.status, 0, sizeof(unsigned int)));
  // about two seconds at the maximum SM clock (clockRate is in kHz)
  int khz = 0;
  if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device_id) != cudaSuccess || khz <= 0) {
    (void)cudaGetLastError();
    khz = 2000000;
  }
  st.spin_budget = 2000ll * khz;
  if (const char* e = std::getenv("FASTNN_B200_SPIN_MS")) {
    const long long ms = std::atoll(e);
    if (ms > 0) st.spin_budget = ms * khz;
  }
  st.ready.store(true, std::memory_order_release);
  return 0;
}

extern "C" int fastnn_cuda_device_count(void) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return count;
}

extern "C" int fastnn_cuda_synchronize(void) {
  FNN_CUDA_OK(cudaDeviceSynchronize());
  return 0;
}

extern "C" void fastnn_cuda_get_memory_info(size_t* free_mem, size_t* total_mem) {
  size_t f = 0, t = 0;
  if (cudaMemGetInfo(&f, &t) != cudaSuccess) (void)cudaGetLastError();
  if (free_mem) *free_mem = f;
  if (total_mem) *total_mem = t;
}

extern "C" int fastnn_cuda_malloc(float** ptr, size_t size) {
  if (ptr == nullptr) return -1;
  FNN_CUDA_OK(cudaMalloc(reinterpret_cast<void**>(ptr), size));
  return 0;
}
extern "C" int fastnn_cuda_free(float* ptr) {
  FNN_CUDA_OK(cudaFree(ptr));
  return 0;
}
extern "C" int fastnn_cuda_memcpy_h2d(float* dst, const float* src, size_t size) {
  FNN_CUDA_OK(cudaMemcpy(dst, src, size, cudaMemcpyHostToDevice));
  return 0;
}
extern "C" int fastnn_cuda_memcpy_d2h(float* dst, const float* src, size_t size) {
  FNN_CUDA_OK(cudaMemcpy(dst, src, size, cudaMemcpyDeviceToHost));
  return 0;
}
extern "C" int fastnn_b200_memcpy_h2d_async(float* dst, const float* src, size_t size, void* stream) {
  if (size == 0) return 0;
  if (dst == nullptr || src == nullptr) return -1;
  FNN_CUDA_OK(cudaMemcpyAsync(dst, src, size, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
  return 0;
}
extern "C" int fastnn_b200_memcpy_d2h_async(float* dst, const float* src, size_t size, void* stream) {
  if (size == 0) return 0;
  if (dst == nullptr || src == nullptr) return -1;
  FNN_CUDA_OK(cudaMemcpyAsync(dst, src, size, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  return 0;
}
extern "C" int fastnn_b200_memcpy_d2d_async(float* dst, const float* src, size_t size, void* stream) {
  if (size == 0) return 0;
  if (dst == nullptr || src == nullptr) return -1;
  FNN_CUDA_OK(cudaMemcpyAsync(dst, src, size, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
  return 0;
}
extern "C" int fastnn_cuda_memcpy_d2d(float* dst, const float* src, size_t size) {
  FNN_CUDA_OK(cudaMemcpy(dst, src, size, cudaMemcpyDeviceToDevice));
  return 0;
}
extern "C" int fastnn_cuda_memset(float* ptr, int value, size_t size) {
  FNN_CUDA_OK(cudaMemset(ptr, value, size));
  return 0;
}

extern "C" int fastnn_cuda_matmul(const float* a, const float* b, float* c, int m, int n, int k,
                                  int lda, int ldb, int ldc, float alpha, float beta) {
  GemmArgs g{FASTNN_B200_NN, a, b, c, m, n, k, 1, lda, ldb, ldc,
             1ll * m * lda, 1ll * k * ldb, 1ll * m * ldc, alpha, beta, nullptr, 0, nullptr};
  return gemm_dispatch(g);
}
extern "C" int fastnn_cuda_matmul_batched(const float* a, const float* b, float* c, int m, int n,
                                          int k, int batch_size, float alpha, float beta) {
  GemmArgs g{FASTNN_B200_NN, a, b, c, m, n, k, batch_size, k, n, n,
             1ll * m * k, 1ll * k * n, 1ll * m * n, alpha, beta, nullptr, 0, nullptr};
  return gemm_dispatch(g);
}
extern "C" int fastnn_cuda_matmul_nt(const float* a, const float* b, float* c, int m, int n, int k) {
  GemmArgs g{FASTNN_B200_NT, a, b, c, m, n, k, 1, k, k, n,
             1ll * m * k, 1ll * n * k, 1ll * m * n, 1.0f, 0.0f, nullptr, 0, nullptr};
  return gemm_dispatch(g);
}
extern "C" int fastnn_cuda_matmul_tn(const float* a, const float* b, float* c, int m, int n, int k) {
  GemmArgs g{FASTNN_B200_TN, a, b, c, m, n, k, 1, m, n, n,
             1ll * k * m, 1ll * k * n, 1ll * m * n, 1.0f, 0.0f, nullptr, 0, nullptr};
  return gemm_dispatch(g);
}
extern "C" int fastnn_cuda_matmul_batched_nt(const float* a, const float* b, float* c, int m, int n,
                                             int k, int batch_size) {
  GemmArgs g{FASTNN_B200_NT, a, b, c, m, n, k, batch_size, k, k, n,
             1ll * m * k, 1ll * n * k, 1ll * m * n, 1.0f, 0.0f, nullptr, 0, nullptr};
  return gemm_dispatch(g);
}
extern "C" int fastnn_cuda_matmul_batched_tn(const float* a, const float* b, float* c, int m, int n,
                                             int k, int batch_size) {
  GemmArgs g{FASTNN_B200_TN, a, b, c, m, n, k, batch_size, m, n, n,
             1ll * k * m, 1ll * k * n, 1ll * m * n, 1.0f, 0.0f, nullptr, 0, nullptr};
  return gemm_dispatch(g);
}

// ================================================================== additions ===

extern "C" int fastnn_b200_gemm_ex(int layout, const float* a, const float* b, float* c, int m,
                                   int n, int k, int batch, long long lda, long long ldb,
                                   long long ldc, long long stride_a, long long stride_b,
                                   long long stride_c, float alpha, float beta, const float* bias,
                                   int act, void* stream) {
  GemmArgs g{layout, a, b, c, m, n, k, batch, lda, ldb, ldc, stride_a, stride_b, stride_c,
             alpha, beta, bias, act, static_cast<cudaStream_t>(stream)};
  return gemm_dispatch(g);
}

extern "C" int fastnn_b200_linear_forward(int layout, const float* x, const float* w,
                                          const float* bias, float* y, int rows, int in_features,
                                          int out_features, int act) {
  if (layout != FASTNN_B200_NT && layout != FASTNN_B200_NN) return -1;
  const long long ldw = (layout == FASTNN_B200_NT) ? in_features : out_features;
  GemmArgs g{layout, x, w, y, rows, out_features, in_features, 1, in_features, ldw, out_features,
             1ll * rows * in_features, 1ll * in_features * out_features, 1ll * rows * out_features,
             1.0f, 0.0f, bias, act, nullptr};
  return gemm_dispatch(g);
}

extern "C" int fastnn_b200_linear_backward_input(int layout, const float* dy, const float* w,
                                                 float* dx, int rows, int out_features,
                                                 int in_features, int act, const float* pre,
                                                 float* bias_grad, void* stream) {
  if (layout != FASTNN_B200_NN && layout != FASTNN_B200_NT) return -1;
  if (rows < 0 || out_features < 0 || in_features < 0 || act < 0 || act > 2) return -1;
  if (act != 0 && pre == nullptr) return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (rows == 0 || in_features == 0) {
    if (bias_grad != nullptr && in_features > 0)
      FNN_CUDA_OK(cudaMemsetAsync(bias_grad, 0, sizeof(float) * in_features, s));
    return 0;
  }
  // NN takes W as Linear stores it, [out, in]; NT takes the transposed copy [in, out]
  const long long ldw = (layout == FASTNN_B200_NN) ? in_features : out_features;
  GemmArgs g{layout, dy, w, dx, rows, in_features, out_features, 1, out_features, ldw, in_features,
             1ll * rows * out_features, 1ll * in_features * out_features, 1ll * rows * in_features,
             1.0f, 0.0f, nullptr, act == 0 ? 0 : act + 2, s};
  g.aux = act == 0 ? nullptr : pre;
  g.ld_aux = in_features;
  g.colsum = bias_grad;
  return gemm_dispatch(g);
}

extern "C" int fastnn_b200_rnn_gates_forward(const float* x_t, long long ld_x, const float* h,
                                             const float* w_ih, const float* w_hh,
                                             const float* b_ih, const float* b_hh, float* gates,
                                             int batch, int input_size, int hidden_size,
                                             int gate_rows, void* stream) {
  if (batch < 0 || input_size < 0 || hidden_size < 0 || gate_rows < 0) return -1;
  if (batch == 0 || gate_rows == 0) return 0;
  if (ld_x < input_size) return -1;
  if (gates == nullptr) return -1;
  if ((input_size > 0 && (x_t == nullptr || w_ih == nullptr)) ||
      (hidden_size > 0 && (h == nullptr || w_hh == nullptr)))
    return -1;
  const float* b1 = b_ih != nullptr ? b_ih : b_hh;          // a single bias goes first
  const float* b2 = b_ih != nullptr ? b_hh : nullptr;
  GemmArgs g{FASTNN_B200_NT, x_t, w_ih, gates, batch, gate_rows, input_size, 1,
             ld_x, input_size, gate_rows, 0, 0, 0, 1.0f, 0.0f, b1, 0,
             static_cast<cudaStream_t>(stream)};
  g.a2 = h; g.b2 = w_hh; g.k2 = hidden_size; g.lda2 = hidden_size; g.ldb2 = hidden_size;
  g.bias2 = b2;
  return dual_dispatch(g);
}

// One launch of the implicit-GEMM convolution kernel (plus its small table / weight pre-passes).
struct ConvCall {
  const float* input;            // [batch, ci, h, w]
  const float* weight;           // as stored; how it is read depends on wmode
  const float* bias;
  float* output;
  int batch, ci, co, h, w;       // input channels and size, output channels, of THIS launch
  int kh, kw;                    // kernel this launch applies
  int sh, sw, ph, pw;            // stride and padding (padding may be negative for a gradient phase)
  int oh, ow;                    // output positions per image
  int dst_h, dst_w, dst_y0, dst_x0, dst_sy, dst_sx;    // where they land (ConvParams)
  int act;
  // 0: weight is [co, ci, kh, kw], used as stored.  1: weight is [ci, co, kh, kw], used with both
  // kernel axes reversed (input gradient of a stride-1 convolution).  2: weight is
  // [ci, co, full_kh, full_kw]; this launch applies the reversed sub-kernel of the taps
  // (ry + wsh * t, rx + wsw * u) -- one phase of a strided input gradient.
  int wmode;
  int full_kh, full_kw, ry, rx, wsh, wsw;
};

static int conv_launch(DeviceState* st, const ConvCall& c, cudaStream_t s) {
  const long long k_ll = 1ll * c.ci * c.kh * c.kw;
  const long long positions = 1ll * c.batch * c.oh * c.ow;
  if (k_ll > (1ll << 30) || positions > (1ll << 40) || positions < 1) return -1;
  const int k = static_cast<int>(k_ll);
  // weights are [co, k] row-major: K-major for the tensor core as they stand.  TMA needs 16-byte
  // rows; otherwise (k = 27 for a 3x3 kernel on RGB) a zero-padded copy goes to the workspace.
  const float* wsrc = c.weight;
  long long w_ld = k;
  const int num_kb = ceil_div(k, fnn::kBlockK);
  const bool copy_w = c.wmode != 0 || (k & 3) != 0 || !aligned16(c.weight);
  const int k_pad = num_kb * fnn::kBlockK;
  // workspace of this stream: [the gather's table, one int4 per k] [padded / flipped weights]
  const size_t tab_bytes = sizeof(int4) * static_cast<size_t>(k_pad);
  const size_t w_bytes = copy_w ? sizeof(float) * static_cast<size_t>(c.co) * k_pad : 0;
  float* ws_ptr = nullptr;
  if (workspace_reserve(st, st->workspaces, s, tab_bytes + w_bytes, &ws_ptr) != 0) return -1;
  int4* ktab = reinterpret_cast<int4*>(ws_ptr);
  if (copy_w) {
    float* wdst = reinterpret_cast<float*>(reinterpret_cast<char*>(ws_ptr) + tab_bytes);
    long long blocks = (1ll * c.co * k_pad + 255) / 256;
    if (blocks > 1024) blocks = 1024;
    if (c.wmode == 1)
      fnn::flip_weights_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(
          c.weight, wdst, c.ci, c.co, c.kh, c.kw, k_pad);
    else if (c.wmode == 2)
      fnn::flip_weights_phase_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(
          c.weight, wdst, c.ci, c.co, c.full_kh, c.full_kw, c.ry, c.rx, c.wsh, c.wsw, c.kh, c.kw, k_pad);
    else
      fnn::pad_weights_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(c.weight, wdst, c.co, k, k_pad);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    wsrc = wdst;
    w_ld = k_pad;
  }
  FNN_CUDA_OK(cudaGetLastError());
  fnn::ConvParams p;
  std::memset(&p, 0, sizeof(p));
  p.batch = c.batch; p.ci = c.ci; p.co = c.co; p.h = c.h; p.w = c.w;
  p.kh = c.kh; p.kw = c.kw; p.sh = c.sh; p.sw = c.sw; p.ph = c.ph; p.pw = c.pw;
  p.oh = c.oh; p.ow = c.ow; p.k = k; p.num_kb = num_kb; p.positions = positions;
  p.dst_h = c.dst_h; p.dst_w = c.dst_w; p.dst_y0 = c.dst_y0; p.dst_x0 = c.dst_x0;
  p.dst_sy = c.dst_sy; p.dst_sx = c.dst_sx;
  p.block_n = c.co >= fnn::kMaxBlockN ? fnn::kMaxBlockN : ceil_div(c.co, 32) * 32;
  // The slab form (input rows of a tile staged in shared memory by TMA) when the rows can be
  // addressed by a tensor map (16-byte row pitch and base), the kernel overhangs the image by at most
  // the four halo columns on either side, and two slabs fit beside four pipeline stages.  (Four
  // stages, no fewer: its four groups of gather warps each take every fourth k-block, and a group
  // that could run more than one use of a stage ahead of the tensor core would mistake the phase of
  // the stage's barrier.)
  CUtensorMap tmX;
  bool slab = false;
  const Tunables& tune = tunables();
  const int plane = c.oh * c.ow;
  if (!tune.conv_no_slab && (c.w & 3) == 0 && aligned16(c.input) && c.w + 2 * fnn::kConvSlabHalo <= 256 &&
      c.pw <= fnn::kConvSlabHalo && (c.ow - 1) * c.sw - c.pw + c.kw - 1 <= c.w - 1 + fnn::kConvSlabHalo &&
      c.pw > -(1 << 20) && c.batch <= 0x7fffffff / ((plane + fnn::kBlockM - 1) / fnn::kBlockM)) {
    const int tiles_pi = (plane + fnn::kBlockM - 1) / fnn::kBlockM;
    int rows_out = 1;                               // output rows one tile can touch
    for (int t = 0; t < tiles_pi; ++t) {
      const int first = t * fnn::kBlockM;
      const int last = first + fnn::kBlockM - 1 < plane ? first + fnn::kBlockM - 1 : plane - 1;
      const int rows = last / c.ow - first / c.ow + 1;
      if (rows > rows_out) rows_out = rows;
    }
    const long long slab_rows = 1ll * (rows_out - 1) * c.sh + c.kh;
    const int pitch = c.w + 2 * fnn::kConvSlabHalo;
    const long long slab_bytes = 1ll * fnn::kConvSlabChannels * slab_rows * pitch * 4;
    const int taps = c.kh * c.kw;
    const long long fixed = 1024 + fnn::kBarrierBytes + ((taps * 128ll + 127) & ~127ll) + 2 * slab_bytes;
    const long long room = static_cast<long long>(kMaxDynSmem) - fixed;
    // stages of the weight tile alone (A lives in tensor memory): four to eight, as many as fit --
    // a stage is only 256 clocks of tensor work, and the ring has to cover the latency of a weight
    // load; channel tiles of at most 128 columns (the A slots take the tensor-memory columns the
    // accumulators leave)
    int slab_bn = p.block_n > 128 ? 128 : p.block_n;
    long long fit = room / (1ll * slab_bn * fnn::kBlockK * 4);
    if (fit < fnn::kConvSlabMinStages) slab_bn = 0;
    const int slab_stages = fit > fnn::kMaxStages ? fnn::kMaxStages : static_cast<int>(fit);
    if (slab_rows <= 256 && slab_bn > 0) {
      const EncodeTiledFn encode = g_encode.load(std::memory_order_acquire);
      cuuint64_t dims[4] = {static_cast<cuuint64_t>(c.w), static_cast<cuuint64_t>(c.h),
                            static_cast<cuuint64_t>(c.ci), static_cast<cuuint64_t>(c.batch)};
      cuuint64_t strides[3] = {c.w * 4ull, 4ull * c.w * c.h, 4ull * c.w * c.h * c.ci};
      cuuint32_t box[4] = {static_cast<cuuint32_t>(pitch), static_cast<cuuint32_t>(slab_rows),
                           static_cast<cuuint32_t>(fnn::kConvSlabChannels), 1};
      cuuint32_t estr[4] = {1, 1, 1, 1};
      if (encode != nullptr && strides[2] < (1ull << 40) &&
          encode(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(c.input), dims, strides, box,
                 estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS) {
        slab = true;
        p.block_n = slab_bn;
        p.tiles_pi = tiles_pi;
        p.taps = taps;
        p.n_chunks = ceil_div(c.ci, fnn::kConvSlabChannels);
        p.slab_rows = static_cast<int>(slab_rows);
        p.slab_pitch = pitch;
        p.slab_bytes = static_cast<int>(slab_bytes);
        p.num_stages = slab_stages;
      }
    }
  }
  const long long tiles_p = slab ? 1ll * c.batch * p.tiles_pi : (positions + fnn::kBlockM - 1) / fnn::kBlockM;
  p.tiles_n = ceil_div(c.co, p.block_n);
  if (tiles_p * p.tiles_n > 0x7fffffffll) return -1;
  p.tiles_p = static_cast<int>(tiles_p);
  p.total_units = static_cast<int>(tiles_p * p.tiles_n);
  if (!slab) {
    const size_t stage = fnn::kStageABytes + static_cast<size_t>(p.block_n) * fnn::kBlockK * 4;
    int stages = static_cast<int>((kMaxDynSmem - 1024 - fnn::kBarrierBytes) / stage);
    p.num_stages = stages > fnn::kMaxStages ? fnn::kMaxStages : stages;
  }
  p.x = c.input; p.ktab = ktab; p.bias = c.bias; p.out = c.output; p.act = c.act;
  p.status = st->status; p.spin_budget = st->spin_budget;
  CUtensorMap tmW;
  if (!encode_map(&tmW, wsrc, static_cast<uint64_t>(w_ld == k ? k : w_ld), c.co, 1, w_ld * 4ull,
                  w_ld * 4ull * c.co, fnn::kBlockK, p.block_n))
    return -1;
  const int grid = p.total_units < st->num_sms ? p.total_units : st->num_sms;
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid, 1, 1);
  // channel tiles of at most 64 columns: the slab form with two MMA-issuing threads
  const bool dual = slab && p.block_n <= 64;
  cfg.blockDim = dim3(dual ? fnn::kConvSlabDualThreads : fnn::kConvThreads, 1, 1);
  cfg.dynamicSmemBytes = slab ? fnn::conv_slab_smem_bytes(p.block_n, p.num_stages, p.slab_bytes, p.taps)
                              : fnn::conv_smem_bytes(p.block_n, p.num_stages);
  cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (dual) {
    FNN_CUDA_OK(cudaLaunchKernelEx(&cfg, fnn::conv2d_tf32_slab_dual_kernel, tmW, tmX, p));
  } else if (slab) {
    FNN_CUDA_OK(cudaLaunchKernelEx(&cfg, fnn::conv2d_tf32_slab_kernel, tmW, tmX, p));
  } else {
    // the global-memory gather reads what depends on k alone from a table written just before
    fnn::conv_ktab_kernel<<<ceil_div(k_pad, 256), 256, 0, s>>>(ktab, k_pad, k, c.kh, c.kw, c.h, c.w);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    FNN_CUDA_OK(cudaLaunchKernelEx(&cfg, fnn::conv2d_tf32_kernel, tmW, p));
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  t_last = LastCall{slab ? 9 : 5, p.block_n, 1, grid};
  return 0;
}

// What the implicit-GEMM gather can encode: (offset inside the image, tap index) in 32 bits and a
// 64-bit tap mask.
static bool conv_gather_covers(int channels, int h, int w, int kh, int kw) {
  return 1ll * kh * kw <= 63 && 1ll * channels * h * w < (1ll << 25);
}

// The convolution.  flip_transpose = false: `weight` is [out, in, kh, kw].  flip_transpose = true:
// `weight` is [in, out, kh, kw] and is used with both kernel axes reversed -- the form in which
// the gradient with respect to the input of a stride-1 convolution is itself a convolution of the
// output gradient.
static int conv_forward_impl(const float* input, const float* weight, const float* bias, float* output,
                             int batch_size, int in_channels, int out_channels, int input_h,
                             int input_w, int kernel_h, int kernel_w, int stride_h, int stride_w,
                             int pad_h, int pad_w, int act, void* stream, bool flip_transpose) {
  if (batch_size < 0 || in_channels < 1 || out_channels < 1 || input_h < 1 || input_w < 1 ||
      kernel_h < 1 || kernel_w < 1 || stride_h < 1 || stride_w < 1 || pad_h < 0 || pad_w < 0 ||
      act < 0 || act > 1)
    return -1;
  if (input_h + 2 * pad_h < kernel_h || input_w + 2 * pad_w < kernel_w) return -1;
  if (batch_size == 0) return 0;
  if (input == nullptr || weight == nullptr || output == nullptr) return -1;
  const int oh = (input_h + 2 * pad_h - kernel_h) / stride_h + 1;      // cuda/kernels.cu:903-904
  const int ow = (input_w + 2 * pad_w - kernel_w) / stride_w + 1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  DeviceState* st = current_state();
  if (st == nullptr) return -1;
  // Kernels of 64 taps or more and images of 2^25 elements or more go to the direct kernel (FP32
  // FMA, one thread per output element): rare shapes, served rather than refused.
  if (!conv_gather_covers(in_channels, input_h, input_w, kernel_h, kernel_w)) {
    const long long total = 1ll * batch_size * oh * ow * out_channels;
    long long blocks = (total + 255) / 256;
    if (blocks > 64ll * st->num_sms) blocks = 64ll * st->num_sms;
    fnn::conv2d_direct_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        input, weight, bias, output, batch_size, in_channels, out_channels, input_h, input_w, kernel_h,
        kernel_w, stride_h, stride_w, pad_h, pad_w, oh, ow, act, flip_transpose ? 1 : 0);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    FNN_CUDA_OK(cudaGetLastError());
    t_last = LastCall{7, 0, 1, static_cast<int>(blocks)};
    return 0;
  }
  ConvCall c;
  std::memset(&c, 0, sizeof(c));
  c.input = input; c.weight = weight; c.bias = bias; c.output = output;
  c.batch = batch_size; c.ci = in_channels; c.co = out_channels; c.h = input_h; c.w = input_w;
  c.kh = kernel_h; c.kw = kernel_w; c.sh = stride_h; c.sw = stride_w; c.ph = pad_h; c.pw = pad_w;
  c.oh = oh; c.ow = ow;
  c.dst_h = oh; c.dst_w = ow; c.dst_y0 = 0; c.dst_x0 = 0; c.dst_sy = 1; c.dst_sx = 1;
  c.act = act; c.wmode = flip_transpose ? 1 : 0;
  return conv_launch(st, c, s);
}

extern "C" int fastnn_b200_conv2d_forward(const float* input, const float* weight, const float* bias,
                                          float* output, int batch_size, int in_channels,
                                          int out_channels, int input_h, int input_w, int kernel_h,
                                          int kernel_w, int stride_h, int stride_w, int pad_h,
                                          int pad_w, int act, void* stream) {
  return conv_forward_impl(input, weight, bias, output, batch_size, in_channels, out_channels, input_h,
                           input_w, kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w, act, stream,
                           false);
}

// grad_input[n, ci, iy, ix] = sum over (co, ki, kj) of grad_output[n, co, iy + ph - ki, ix + pw - kj]
// * weight[co, ci, ki, kj] for a stride-1 convolution: with ki' = kh-1-ki this is the forward
// kernel run on grad_output (co channels in, ci out) with the kernel reversed and padding
// kh-1-ph.
// Stride (sh, sw): input row iy receives only the taps ki = ry + sh * t with ry = (iy + ph) % sh,
// from output row (iy + ph - ki) / sh.  The rows of one residue ry (and columns of one rx) form a
// PHASE, and a phase is again a stride-1 convolution of grad_output -- with the reversed sub-kernel
// of those taps -- whose results land on every sh-th row and sw-th column of grad_input.  So the
// gradient is sh * sw launches of the same implicit-GEMM kernel, no multiplication by a zero, no
// column matrix, no atomics (what FastNN's GEMM + col2im computes, cuda/kernels.cu:862-893,
// 949-987).  Phases no tap reaches (stride larger than the kernel) are zeros.
// Shapes the gather cannot encode fall back to the gather-form FP32 kernel.
extern "C" int fastnn_b200_conv2d_backward_data(const float* grad_output, const float* weight,
                                                float* grad_input, int batch_size, int in_channels,
                                                int out_channels, int input_h, int input_w,
                                                int output_h, int output_w, int kernel_h,
                                                int kernel_w, int stride_h, int stride_w, int pad_h,
                                                int pad_w, void* stream) {
  if (batch_size < 0 || in_channels < 1 || out_channels < 1 || input_h < 1 || input_w < 1 ||
      kernel_h < 1 || kernel_w < 1 || stride_h < 1 || stride_w < 1 || pad_h < 0 || pad_w < 0)
    return -1;
  if (input_h + 2 * pad_h < kernel_h || input_w + 2 * pad_w < kernel_w) return -1;
  if (output_h != (input_h + 2 * pad_h - kernel_h) / stride_h + 1 ||
      output_w != (input_w + 2 * pad_w - kernel_w) / stride_w + 1)
    return -1;
  if (stride_h == 1 && stride_w == 1 && pad_h <= kernel_h - 1 && pad_w <= kernel_w - 1)
    return conv_forward_impl(grad_output, weight, nullptr, grad_input, batch_size, out_channels,
                             in_channels, output_h, output_w, kernel_h, kernel_w, 1, 1,
                             kernel_h - 1 - pad_h, kernel_w - 1 - pad_w, 0, stream, true);
  if (batch_size == 0) return 0;
  if (grad_output == nullptr || weight == nullptr || grad_input == nullptr) return -1;
  DeviceState* st = current_state();
  if (st == nullptr) return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long total = 1ll * batch_size * in_channels * input_h * input_w;
  if (conv_gather_covers(out_channels, output_h, output_w, kernel_h, kernel_w) && t_policy.policy != 1) {
    if (stride_h > kernel_h || stride_w > kernel_w)        // some phases get no tap at all
      FNN_CUDA_OK(cudaMemsetAsync(grad_input, 0, sizeof(float) * total, s));
    for (int ry = 0; ry < stride_h && ry < kernel_h; ++ry) {
      const int ty = (kernel_h - ry + stride_h - 1) / stride_h;             // taps ki = ry, ry + sh, ...
      const int iy_first = ((ry - pad_h) % stride_h + stride_h) % stride_h; // first input row of the phase
      if (iy_first >= input_h) continue;
      const int rows = (input_h - 1 - iy_first) / stride_h + 1;
      const int a_min = (iy_first + pad_h - ry) / stride_h;                 // its (iy + ph - ry) / sh
      for (int rx = 0; rx < stride_w && rx < kernel_w; ++rx) {
        const int tx = (kernel_w - rx + stride_w - 1) / stride_w;
        const int ix_first = ((rx - pad_w) % stride_w + stride_w) % stride_w;
        if (ix_first >= input_w) continue;
        const int cols = (input_w - 1 - ix_first) / stride_w + 1;
        const int b_min = (ix_first + pad_w - rx) / stride_w;
        ConvCall c;
        std::memset(&c, 0, sizeof(c));
        c.input = grad_output; c.weight = weight; c.bias = nullptr; c.output = grad_input;
        c.batch = batch_size; c.ci = out_channels; c.co = in_channels; c.h = output_h; c.w = output_w;
        c.kh = ty; c.kw = tx; c.sh = 1; c.sw = 1;
        c.ph = ty - 1 - a_min; c.pw = tx - 1 - b_min;       // may be negative: the gather only tests bounds
        c.oh = rows; c.ow = cols;
        c.dst_h = input_h; c.dst_w = input_w; c.dst_y0 = iy_first; c.dst_x0 = ix_first;
        c.dst_sy = stride_h; c.dst_sx = stride_w;
        c.act = 0; c.wmode = 2;
        c.full_kh = kernel_h; c.full_kw = kernel_w; c.ry = ry; c.rx = rx; c.wsh = stride_h; c.wsw = stride_w;
        const int rc = conv_launch(st, c, s);
        if (rc != 0) return rc;
      }
    }
    return 0;
  }
  long long blocks = (total + 255) / 256;
  if (blocks > 64ll * st->num_sms) blocks = 64ll * st->num_sms;
  fnn::conv2d_backward_data_direct_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(
      grad_output, weight, grad_input, batch_size, in_channels, out_channels, input_h, input_w, output_h,
      output_w, kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  FNN_CUDA_OK(cudaGetLastError());
  t_last = LastCall{7, 0, 1, static_cast<int>(blocks)};
  return 0;
}

// FastNN's own entry (cuda/kernels.cu:949-987): same arguments, default stream.
extern "C" int fastnn_cuda_conv2d_backward_data(const float* grad_output, const float* weight,
                                                float* grad_input, int batch_size, int in_channels,
                                                int out_channels, int input_h, int input_w,
                                                int output_h, int output_w, int kernel_h,
                                                int kernel_w, int stride_h, int stride_w, int pad_h,
                                                int pad_w) {
  return fastnn_b200_conv2d_backward_data(grad_output, weight, grad_input, batch_size, in_channels,
                                          out_channels, input_h, input_w, output_h, output_w, kernel_h,
                                          kernel_w, stride_h, stride_w, pad_h, pad_w, nullptr);
}

// grad_weight[co, k] = sum over images n and positions p of grad_output[n, co, p] * col[n, k, p].
// Implicit GEMM (conv_wgrad_tcgen05.cuh): grad_output tiles by TMA, the column values gathered
// straight into the B stages, the contraction over all positions of all images cut into slices so
// that every SM has a unit; slices are added in order by the split-K reduce kernel.  Needs
// out_h * out_w to be a multiple of 4 (16-byte rows of grad_output for TMA).
// The weight gradient with the gathered operand in tensor memory (conv_wgrad_slab_tcgen05.cuh).
// Returns 1 when the shape is outside that form's conditions (the caller then takes another form):
// input rows a tensor map can address (16-byte pitch and base, at most 244 columns), the kernel
// overhanging the image by at most four columns on either side, output rows of 16-byte pitch, and
// two slabs beside at least four stages of dY tiles in shared memory.
static int conv_wgrad_slab(DeviceState* st, const float* input, const float* grad_output, float* grad_weight,
                           int batch_size, int in_channels, int out_channels, int input_h, int input_w,
                           int output_h, int output_w, int kernel_h, int kernel_w, int stride_h, int stride_w,
                           int pad_h, int pad_w, int k, cudaStream_t s) {
  const Tunables& tune = tunables();
  if (tune.conv_no_slab) return 1;
  const int pitch = input_w + 12;            // four halo columns either side + four that keep rows off one bank
  if ((input_w & 3) != 0 || !aligned16(input) || pitch > 256 || pad_w > fnn::kWgradSlabHalo || stride_w > 4 ||
      (output_w - 1) * stride_w - pad_w + kernel_w - 1 > input_w - 1 + fnn::kWgradSlabHalo ||
      (output_w & 3) != 0 || !aligned16(grad_output) || out_channels > (1 << 20))
    return 1;
  fnn::WgradSlabParams p;
  std::memset(&p, 0, sizeof(p));
  p.batch = batch_size; p.ci = in_channels; p.co = out_channels; p.h = input_h; p.w = input_w;
  p.kh = kernel_h; p.kw = kernel_w; p.sh = stride_h; p.sw = stride_w; p.ph = pad_h; p.pw = pad_w;
  p.oh = output_h; p.ow = output_w; p.k_taps = k; p.taps = kernel_h * kernel_w;
  p.tiles_m = ceil_div(k, fnn::kBlockM);
  p.block_n = out_channels >= 128 ? 128 : ceil_div(out_channels, 32) * 32;
  p.tiles_n = ceil_div(out_channels, p.block_n);
  p.kb_per_row = ceil_div(output_w, fnn::kBlockK);
  p.slab_ch = (fnn::kBlockM - 1) / p.taps + 2;          // channels 128 consecutive taps can touch
  if (p.slab_ch > 256) return 1;
  p.slab_pitch = pitch;
  const size_t stage = static_cast<size_t>(p.block_n) * fnn::kBlockK * 4;
  // output rows per slab: as many as keep two slabs beside four stages
  const long long budget = static_cast<long long>(kMaxDynSmem) - 1024 - fnn::kBarrierBytes - fnn::kWgradSlabTailBytes -
                           4 * static_cast<long long>(stage);
  p.g_rows = 0;
  for (int g : {8, 4, 2, 1}) {
    const long long rows = 1ll * (g - 1) * stride_h + kernel_h;
    const long long bytes = 1ll * p.slab_ch * rows * pitch * 4;
    if (rows <= 256 && 2 * bytes <= budget && bytes <= 48 * 1024) {
      p.g_rows = g > output_h ? output_h : g;
      p.slab_rows = static_cast<int>(1ll * (p.g_rows - 1) * stride_h + kernel_h);
      p.slab_bytes = static_cast<int>(1ll * p.slab_ch * p.slab_rows * pitch * 4);
      break;
    }
  }
  if (p.g_rows == 0) return 1;
  p.slabs_per_image = ceil_div(output_h, p.g_rows);
  if (1ll * batch_size * p.slabs_per_image > 0x7fffffffll) return 1;
  p.total_slabs = batch_size * p.slabs_per_image;
  const long long room = static_cast<long long>(kMaxDynSmem) - 1024 - fnn::kBarrierBytes - fnn::kWgradSlabTailBytes -
                         2ll * p.slab_bytes;
  long long stages = room / static_cast<long long>(stage);
  if (stages < 4) return 1;
  p.num_stages = stages > fnn::kMaxStages ? fnn::kMaxStages : static_cast<int>(stages);
  long long slices = st->num_sms / (1ll * p.tiles_m * p.tiles_n);
  if (slices > p.total_slabs) slices = p.total_slabs;
  if (slices < 1) slices = 1;
  p.slices = static_cast<int>(slices);
  const long long units = 1ll * p.tiles_m * p.tiles_n * p.slices;
  if (units > 0x7fffffffll) return 1;
  p.total_units = static_cast<int>(units);
  const size_t part_floats = p.slices > 1 ? static_cast<size_t>(p.slices) * out_channels * k : 0;
  float* partials = nullptr;
  if (part_floats > 0 && workspace_reserve(st, st->conv_ws, s, sizeof(float) * part_floats, &partials) != 0) return -1;
  p.partial = p.slices > 1 ? partials : grad_weight;
  p.status = st->status; p.spin_budget = st->spin_budget;
  const EncodeTiledFn encode = g_encode.load(std::memory_order_acquire);
  if (encode == nullptr) return 1;
  CUtensorMap tmG, tmX;
  {
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(output_w), static_cast<cuuint64_t>(output_h),
                          static_cast<cuuint64_t>(out_channels), static_cast<cuuint64_t>(batch_size)};
    cuuint64_t strides[3] = {output_w * 4ull, 4ull * output_w * output_h, 4ull * output_w * output_h * out_channels};
    cuuint32_t box[4] = {static_cast<cuuint32_t>(fnn::kBlockK), 1, static_cast<cuuint32_t>(p.block_n), 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (strides[2] >= (1ull << 40) ||
        encode(&tmG, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(grad_output), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return 1;
  }
  {
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(input_w), static_cast<cuuint64_t>(input_h),
                          static_cast<cuuint64_t>(in_channels), static_cast<cuuint64_t>(batch_size)};
    cuuint64_t strides[3] = {input_w * 4ull, 4ull * input_w * input_h, 4ull * input_w * input_h * in_channels};
    cuuint32_t box[4] = {static_cast<cuuint32_t>(pitch), static_cast<cuuint32_t>(p.slab_rows),
                         static_cast<cuuint32_t>(p.slab_ch), 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (strides[2] >= (1ull << 40) ||
        encode(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(input), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return 1;
  }
  const int grid = p.total_units < st->num_sms ? p.total_units : st->num_sms;
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(fnn::kWgradSlabThreads, 1, 1);
  cfg.dynamicSmemBytes = fnn::wgrad_slab_smem_bytes(p.block_n, p.num_stages, p.slab_bytes);
  cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  FNN_CUDA_OK(cudaLaunchKernelEx(&cfg, fnn::conv2d_wgrad_slab_kernel, tmG, tmX, p));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (p.slices > 1) {
    const long long total = 1ll * out_channels * k;
    const bool vec = (k & 3) == 0 && aligned16(grad_weight) && aligned16(partials);
    long long rblocks = ((vec ? total / 4 : total) + 255) / 256;
    if (rblocks > 8ll * st->num_sms) rblocks = 8ll * st->num_sms;
    if (rblocks < 1) rblocks = 1;
    if (vec)
      fnn::splitk_reduce_vec4_kernel<<<static_cast<unsigned>(rblocks), 256, 0, s>>>(
          reinterpret_cast<const float4*>(partials), grad_weight, nullptr, out_channels, k, 1, p.slices, k, total,
          1.0f, 0.0f, 0);
    else
      fnn::splitk_reduce_kernel<<<static_cast<unsigned>(rblocks), 256, 0, s>>>(
          partials, grad_weight, nullptr, out_channels, k, 1, p.slices, k, total, 1.0f, 0.0f, 0);
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  FNN_CUDA_OK(cudaGetLastError());
  t_last = LastCall{11, p.block_n, p.slices, grid};
  return 0;
}

static int conv_wgrad_implicit(DeviceState* st, const float* input, const float* grad_output, float* grad_weight,
                               int batch_size, int in_channels, int out_channels, int input_h, int input_w,
                               int output_h, int output_w, int kernel_h, int kernel_w, int stride_h,
                               int stride_w, int pad_h, int pad_w, int k, cudaStream_t s) {
  fnn::WgradParams p;
  std::memset(&p, 0, sizeof(p));
  p.batch = batch_size; p.ci = in_channels; p.co = out_channels; p.h = input_h; p.w = input_w;
  p.kh = kernel_h; p.kw = kernel_w; p.sh = stride_h; p.sw = stride_w; p.ph = pad_h; p.pw = pad_w;
  p.oh = output_h; p.ow = output_w; p.k = k; p.plane = output_h * output_w;
  p.kb_per_image = ceil_div(p.plane, fnn::kBlockK);
  p.total_kb = 1ll * batch_size * p.kb_per_image;
  // tap tiles: equal widths, multiples of 64 (the gather warps take rows in groups of four)
  const int n64 = ceil_div(k, 64) * 64;
  p.tiles_n = ceil_div(n64, fnn::kMaxBlockN);
  p.block_n = ceil_div(ceil_div(n64, p.tiles_n), 64) * 64;
  p.tiles_m = ceil_div(out_channels, fnn::kBlockM);
  // slices: one unit per SM when the tiles alone are fewer, at least eight k-blocks each
  long long slices = st->num_sms / (1ll * p.tiles_m * p.tiles_n);
  if (slices > p.total_kb / 8) slices = p.total_kb / 8;
  if (slices < 1) slices = 1;
  p.kb_per_slice = (p.total_kb + slices - 1) / slices;
  p.slices = static_cast<int>((p.total_kb + p.kb_per_slice - 1) / p.kb_per_slice);   // none empty
  const long long units = 1ll * p.tiles_m * p.tiles_n * p.slices;
  if (units > 0x7fffffffll) return -1;
  p.total_units = static_cast<int>(units);
  const size_t stage = fnn::kStageABytes + static_cast<size_t>(p.block_n) * fnn::kBlockK * 4;
  const int stages = static_cast<int>((kMaxDynSmem - 1024 - fnn::kBarrierBytes - fnn::kWgradTableBytes) / stage);
  p.num_stages = stages > fnn::kMaxStages ? fnn::kMaxStages : stages;
  // this stream's scratch: [tap table] [partial sums of the slices]
  const size_t tab_entries = static_cast<size_t>(p.tiles_n) * p.block_n;
  const size_t tab_bytes = sizeof(int4) * tab_entries;
  const size_t part_floats = p.slices > 1 ? static_cast<size_t>(p.slices) * out_channels * k : 0;
  float* ws = nullptr;
  if (workspace_reserve(st, st->conv_ws, s, tab_bytes + sizeof(float) * part_floats, &ws) != 0) return -1;
  int4* ktab = reinterpret_cast<int4*>(ws);
  float* partials = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + tab_bytes);
  fnn::wgrad_ktab_kernel<<<ceil_div(static_cast<int>(tab_entries), 256), 256, 0, s>>>(
      ktab, static_cast<int>(tab_entries), k, kernel_h, kernel_w, input_h, input_w);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  FNN_CUDA_OK(cudaGetLastError());
  p.x = input; p.ktab = ktab; p.out = p.slices > 1 ? partials : grad_weight;
  p.status = st->status; p.spin_budget = st->spin_budget;
  CUtensorMap tmG;
  const uint64_t plane = static_cast<uint64_t>(p.plane);
  if (!encode_map(&tmG, grad_output, plane, out_channels, batch_size, plane * 4ull,
                  plane * 4ull * out_channels, fnn::kBlockK, fnn::kBlockM))
    return -1;
  const int grid = p.total_units < st->num_sms ? p.total_units : st->num_sms;
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(fnn::kWgradThreads, 1, 1);
  cfg.dynamicSmemBytes = fnn::wgrad_smem_bytes(p.block_n, p.num_stages);
  cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  FNN_CUDA_OK(cudaLaunchKernelEx(&cfg, fnn::conv2d_wgrad_tf32_kernel, tmG, p));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (p.slices > 1) {
    const long long total = 1ll * out_channels * k;
    const bool vec = (k & 3) == 0 && aligned16(grad_weight) && aligned16(partials);
    long long rblocks = ((vec ? total / 4 : total) + 255) / 256;
    if (rblocks > 8ll * st->num_sms) rblocks = 8ll * st->num_sms;
    if (rblocks < 1) rblocks = 1;
    if (vec)
      fnn::splitk_reduce_vec4_kernel<<<static_cast<unsigned>(rblocks), 256, 0, s>>>(
          reinterpret_cast<const float4*>(partials), grad_weight, nullptr, out_channels, k, 1, p.slices, k, total,
          1.0f, 0.0f, 0);
    else
      fnn::splitk_reduce_kernel<<<static_cast<unsigned>(rblocks), 256, 0, s>>>(
          partials, grad_weight, nullptr, out_channels, k, 1, p.slices, k, total, 1.0f, 0.0f, 0);
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  FNN_CUDA_OK(cudaGetLastError());
  t_last = LastCall{5, p.block_n, p.slices, grid};
  return 0;
}

// The explicit form, kept for outputs whose plane is not a multiple of four positions: one
// im2col launch for all images (tap-major, positions contiguous), one batched NT GEMM
// grad_output[n] . col[n]^T into per-image partials -- both operands contiguous along the
// contraction -- and one fixed-order sum over the images.
extern "C" int fastnn_b200_conv2d_backward_weight(const float* input, const float* grad_output,
                                                  float* grad_weight, int batch_size, int in_channels,
                                                  int out_channels, int input_h, int input_w,
                                                  int output_h, int output_w, int kernel_h,
                                                  int kernel_w, int stride_h, int stride_w, int pad_h,
                                                  int pad_w, void* stream) {
  if (batch_size < 0 || in_channels < 1 || out_channels < 1 || input_h < 1 || input_w < 1 ||
      kernel_h < 1 || kernel_w < 1 || stride_h < 1 || stride_w < 1 || pad_h < 0 || pad_w < 0)
    return -1;
  if (input_h + 2 * pad_h < kernel_h || input_w + 2 * pad_w < kernel_w) return -1;
  if (output_h != (input_h + 2 * pad_h - kernel_h) / stride_h + 1 ||
      output_w != (input_w + 2 * pad_w - kernel_w) / stride_w + 1)
    return -1;
  if (grad_weight == nullptr) return -1;
  const long long k_ll = 1ll * in_channels * kernel_h * kernel_w;
  const long long plane = 1ll * output_h * output_w;
  if (k_ll > (1ll << 24) || plane > (1ll << 24) || 1ll * batch_size * plane * k_ll > (1ll << 34)) return -1;
  const int k = static_cast<int>(k_ll);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (batch_size == 0) {
    FNN_CUDA_OK(cudaMemsetAsync(grad_weight, 0, sizeof(float) * out_channels * k_ll, s));
    return 0;
  }
  if (input == nullptr || grad_output == nullptr) return -1;
  {
    DeviceState* st0 = current_state();
    if (st0 == nullptr) return -1;
    if (t_policy.policy != 1) {
      const int rc = conv_wgrad_slab(st0, input, grad_output, grad_weight, batch_size, in_channels, out_channels,
                                     input_h, input_w, output_h, output_w, kernel_h, kernel_w, stride_h, stride_w,
                                     pad_h, pad_w, k, s);
      if (rc <= 0) return rc;
    }
    if ((plane & 3) == 0 && aligned16(grad_output) && 1ll * in_channels * input_h * input_w < (1ll << 30) &&
        t_policy.policy != 1)
      return conv_wgrad_implicit(st0, input, grad_output, grad_weight, batch_size, in_channels, out_channels,
                                 input_h, input_w, output_h, output_w, kernel_h, kernel_w, stride_h, stride_w,
                                 pad_h, pad_w, k, s);
  }
  const int ldp = ceil_div(static_cast<int>(plane), 4) * 4;      // 16-byte rows for TMA
  const size_t col_floats = static_cast<size_t>(batch_size) * k * ldp;
  const size_t part_floats = static_cast<size_t>(batch_size) * out_channels * k;
  float* col = nullptr;
  DeviceState* st = current_state();
  if (st == nullptr) return -1;
  const int num_sms = st->num_sms;
  if (workspace_reserve(st, st->conv_ws, s, sizeof(float) * (col_floats + part_floats + 64), &col) != 0)
    return -1;
  float* partials = col + ((col_floats + 63) / 64) * 64;  // keeps the 16-byte alignment
  long long blocks = (1ll * batch_size * k + 3) / 4;               // four rows of col per block and turn
  if (blocks > 32ll * num_sms) blocks = 32ll * num_sms;
  fnn::im2col_taps_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(
      input, col, batch_size, in_channels, input_h, input_w, kernel_h, kernel_w, stride_h, stride_w, pad_h,
      pad_w, output_h, output_w, ldp);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  FNN_CUDA_OK(cudaGetLastError());
  // per image: partial[n][co, k] = grad_output[n][co, P] . col[n][k, P]^T
  GemmArgs g{FASTNN_B200_NT, grad_output, col, partials, out_channels, k, static_cast<int>(plane),
             batch_size, plane, ldp, k, 1ll * out_channels * plane, 1ll * k * ldp, 1ll * out_channels * k,
             1.0f, 0.0f, nullptr, 0, s};
  g.force_split_k = 1;
  const int rc = gemm_dispatch(g);
  if (rc != 0) return rc;
  const long long total = 1ll * out_channels * k;
  long long rblocks = (total + 255) / 256;
  if (rblocks > 8ll * num_sms) rblocks = 8ll * num_sms;
  fnn::splitk_reduce_kernel<<<static_cast<unsigned>(rblocks), 256, 0, s>>>(
      partials, grad_weight, nullptr, out_channels, k, 1, batch_size, k, total, 1.0f, 0.0f, 0);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  FNN_CUDA_OK(cudaGetLastError());
  return 0;
}

// FastNN's own entry (cuda/kernels.cu:989-1026): same arguments, default stream.
extern "C" int fastnn_cuda_conv2d_backward_weight(const float* input, const float* grad_output,
                                                  float* grad_weight, int batch_size, int in_channels,
                                                  int out_channels, int input_h, int input_w,
                                                  int output_h, int output_w, int kernel_h,
                                                  int kernel_w, int stride_h, int stride_w, int pad_h,
                                                  int pad_w) {
  return fastnn_b200_conv2d_backward_weight(input, grad_output, grad_weight, batch_size, in_channels,
                                            out_channels, input_h, input_w, output_h, output_w, kernel_h,
                                            kernel_w, stride_h, stride_w, pad_h, pad_w, nullptr);
}

// FastNN's own entry (cuda/kernels.cu:896-946): same arguments, default stream, no activation.
extern "C" int fastnn_cuda_conv2d_forward(const float* input, const float* weight, const float* bias,
                                          float* output, int batch_size, int in_channels,
                                          int out_channels, int input_h, int input_w, int kernel_h,
                                          int kernel_w, int stride_h, int stride_w, int pad_h,
                                          int pad_w) {
  return fastnn_b200_conv2d_forward(input, weight, bias, output, batch_size, in_channels, out_channels,
                                    input_h, input_w, kernel_h, kernel_w, stride_h, stride_w, pad_h,
                                    pad_w, 0, nullptr);
}

// The attention core for every shape: the fused kernel when it covers the call and the caller
// does not want the probabilities, else FastNN's own composition on this library's GEMMs --
// batched scale * Q.K^T, masked row softmax in place, batched P.V.
static int attention_impl(const float* q, const float* k, const float* v, float* o, float* attn_weights,
                          const float* mask, int batch_heads, int t_q, int t_k, int head_dim, float scale,
                          int causal, void* stream) {
  if (batch_heads < 0 || t_q < 0 || t_k < 1 || head_dim < 1) return -1;
  if (batch_heads == 0 || t_q == 0) return 0;
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr) return -1;
  DeviceState* st = current_state();
  if (st == nullptr) return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int tk_pad = ceil_div(t_k, 32) * 32;
  // Q/K/V sets in flight per CTA: a set is held from its load until P.V has read V, so the loads
  // of later units need sets of their own to run ahead; as many as fit, up to four.
  int nsets = fnn::kAttnMaxSets;
  fnn::AttnSmem plan;
  std::memset(&plan, 0, sizeof(plan));
  bool fused = attn_weights == nullptr && (head_dim % 32) == 0 && head_dim <= 128 && t_k <= 256 &&
               scale > 0.0f && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(o) &&
               1ll * batch_heads * ceil_div(t_q, 128) <= 0x7fffffffll;
  if (fused) {
    plan = fnn::attn_smem_plan(head_dim, tk_pad, nsets);
    while (plan.total > kMaxDynSmem && nsets > 1) plan = fnn::attn_smem_plan(head_dim, tk_pad, --nsets);
    fused = plan.total <= kMaxDynSmem;
  }
  if (!fused) {
    // scores: the caller's attn_weights, or this stream's scratch
    const long long rows = 1ll * batch_heads * t_q;
    if (rows * t_k > (1ll << 40)) return -1;
    float* scores = attn_weights;
    if (scores == nullptr &&
        workspace_reserve(st, st->attn_ws, s, sizeof(float) * static_cast<size_t>(rows) * t_k, &scores) != 0)
      return -1;
    GemmArgs g1{FASTNN_B200_NT, q, k, scores, t_q, t_k, head_dim, batch_heads, head_dim, head_dim, t_k,
                1ll * t_q * head_dim, 1ll * t_k * head_dim, 1ll * t_q * t_k, scale, 0.0f, nullptr, 0, s};
    int rc = gemm_dispatch(g1);
    if (rc != 0) return rc;
    long long blocks = (rows + 7) / 8;                       // eight rows (warps) per block
    if (blocks > 32ll * st->num_sms) blocks = 32ll * st->num_sms;
    fnn::masked_softmax_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(scores, mask, rows, t_q, t_k,
                                                                                causal ? 1 : 0);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    FNN_CUDA_OK(cudaGetLastError());
    GemmArgs g2{FASTNN_B200_NN, scores, v, o, t_q, head_dim, t_k, batch_heads, t_k, head_dim, head_dim,
                1ll * t_q * t_k, 1ll * t_k * head_dim, 1ll * t_q * head_dim, 1.0f, 0.0f, nullptr, 0, s};
    rc = gemm_dispatch(g2);
    if (rc == 0) t_last.path = 8;
    return rc;
  }
  fnn::AttnParams p;
  std::memset(&p, 0, sizeof(p));
  p.heads = batch_heads; p.tq = t_q; p.tk = t_k; p.d = head_dim; p.tk_pad = tk_pad;
  p.q_tiles = ceil_div(t_q, 128);
  p.total_units = static_cast<int>(1ll * batch_heads * p.q_tiles);
  p.scale = scale; p.causal = causal ? 1 : 0; p.nsets = nsets; p.mask = mask;
  p.status = st->status; p.spin_budget = st->spin_budget;
  CUtensorMap tmQ, tmK, tmV, tmO;
  const uint64_t D = head_dim, H = batch_heads;
  bool ok = encode_map(&tmQ, q, D, t_q, H, D * 4ull, D * 4ull * t_q, 32, 128);
  ok = ok && encode_map(&tmK, k, D, t_k, H, D * 4ull, D * 4ull * t_k, 32, tk_pad);
  ok = ok && encode_map(&tmV, v, D, t_k, H, D * 4ull, D * 4ull * t_k, 32, tk_pad, true);
  ok = ok && encode_map(&tmO, o, D, t_q, H, D * 4ull, D * 4ull * t_q, 32, 32);
  if (!ok) return -1;
  const int grid = p.total_units < st->num_sms ? p.total_units : st->num_sms;
  {
    // launched as a programmatic dependent, like the single-CTA GEMM: set-up overlaps the tail of
    // the previous kernel of the stream, global memory is touched only after griddepcontrol.wait
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(fnn::kAttnThreads, 1, 1);
    cfg.dynamicSmemBytes = plan.total;
    cfg.stream = s;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    FNN_CUDA_OK(cudaLaunchKernelEx(&cfg, fnn::attention_tf32_kernel, tmQ, tmK, tmV, tmO, p));
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  FNN_CUDA_OK(cudaGetLastError());
  t_last = LastCall{4, tk_pad, 1, grid};
  return 0;
}

extern "C" int fastnn_b200_attention_forward(const float* q, const float* k, const float* v, float* o,
                                             int batch_heads, int t_q, int t_k, int head_dim,
                                             float scale, int causal, void* stream) {
  return attention_impl(q, k, v, o, nullptr, nullptr, batch_heads, t_q, t_k, head_dim, scale, causal, stream);
}

extern "C" int fastnn_b200_attention_forward_ex(const float* q, const float* k, const float* v, float* o,
                                                float* attn_weights, const float* mask, int batch_heads,
                                                int t_q, int t_k, int head_dim, float scale, int causal,
                                                void* stream) {
  return attention_impl(q, k, v, o, attn_weights, mask, batch_heads, t_q, t_k, head_dim, scale, causal, stream);
}

// FastNN's own entry (cuda/kernels.cu:1707-1776): same arguments, default stream.  There the
// causal flag and the mask are accepted and ignored (the masking code is dead); here both work.
extern "C" int fastnn_cuda_scaled_dot_product_attention(const float* query, const float* key,
                                                        const float* value, float* output,
                                                        float* attn_weights, const float* mask,
                                                        int batch_size, int num_heads, int seq_len_q,
                                                        int seq_len_k, int head_dim, float scale,
                                                        int causal) {
  if (batch_size < 0 || num_heads < 0 || 1ll * batch_size * num_heads > 0x7fffffffll) return -1;
  return attention_impl(query, key, value, output, attn_weights, mask, batch_size * num_heads, seq_len_q,
                        seq_len_k, head_dim, scale, causal, nullptr);
}

extern "C" int fastnn_b200_reduce_partials(const float* partials, float* c, int m, int n, int count,
                                           long long ldc, float alpha, float beta,
                                           const float* bias, int act, void* stream) {
  if (m < 0 || n < 0 || count < 1 || act < 0 || act > 2 || ldc < n) return -1;
  if (m == 0 || n == 0) return 0;
  if (partials == nullptr || c == nullptr) return -1;
  DeviceState* st = current_state();
  if (st == nullptr) return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long total = 1ll * m * n;
  const bool vec = (n & 3) == 0 && aligned16(partials) && aligned16(c) && (ldc & 3) == 0 &&
                   (bias == nullptr || aligned16(bias));
  long long blocks = ((vec ? total / 4 : total) + 255) / 256;
  if (blocks > 8ll * st->num_sms) blocks = 8ll * st->num_sms;
  if (blocks < 1) blocks = 1;
  if (vec)
    fnn::splitk_reduce_vec4_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        reinterpret_cast<const float4*>(partials), c, bias, m, n, 1, count, ldc, total, alpha, beta, act);
  else
    fnn::splitk_reduce_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        partials, c, bias, m, n, 1, count, ldc, total, alpha, beta, act);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  FNN_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int fastnn_b200_set_policy(int policy, int block_n, int split_k) {
  if (policy < 0 || policy > 6) return -1;
  if (block_n < 0 || (block_n % 32) != 0) return -1;
  if (block_n > fnn::kMaxBlockN && !(policy == 4 && block_n == fnn::kPairWideBlockN)) return -1;
  if (split_k < 0) return -1;
  t_policy.policy = policy;
  t_policy.block_n = block_n;
  t_policy.split_k = split_k;
  return 0;
}

extern "C" int fastnn_b200_last_path(int* block_n, int* split_k, int* num_ctas) {
  if (block_n) *block_n = t_last.block_n;
  if (split_k) *split_k = t_last.split_k;
  if (num_ctas) *num_ctas = t_last.num_ctas;
  return t_last.path;
}

// The planner's choice for a GEMM, without launching anything.  With no initialised device the
// figures of a B200 stand in (148 SMs, 74 CTA pairs, clusters as measured there), so the host
// logic can be exercised on a machine without a GPU.
extern "C" int fastnn_b200_plan_query(int layout, int m, int n, int k, int batch, int* block_n,
                                      int* split_k, int* cta_pair, int* cluster_k) {
  if (layout < 0 || layout > 2 || m < 1 || n < 1 || k < 1 || batch < 1) return -1;
  int num_sms = 148, max_clusters = 74;
  int slots[5] = {0, 148, 132, 120, 112}, slots_half[5] = {0, 148, 132, 120, 112};   // as a B200 reports
  {
    int dev = -1;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices &&
        g_dev[dev].ready.load(std::memory_order_acquire)) {
      num_sms = g_dev[dev].num_sms;
      max_clusters = g_dev[dev].max_clusters;
      for (int i = 0; i < 5; ++i) { slots[i] = g_dev[dev].ck_slots[i]; slots_half[i] = g_dev[dev].ck_slots_half[i]; }
    } else {
      (void)cudaGetLastError();
    }
  }
  const bool a_mn = layout == FASTNN_B200_TN && (m % 32) != 0;
  const bool b_mn = layout != FASTNN_B200_NT && (n % 32) != 0;
  Plan plan = choose_plan(m, n, k, batch, num_sms, max_clusters, a_mn, b_mn, 0, slots, slots_half);
  refine_large_plan(&plan, m, n, k, batch, num_sms, max_clusters, a_mn, b_mn, 0, false, !tunables().no_wide);
  if (block_n) *block_n = plan.block_n;
  if (split_k) *split_k = plan.split_k;
  if (cta_pair) *cta_pair = plan.pair ? 1 : 0;
  if (cluster_k) *cluster_k = plan.cluster_k ? 1 : 0;
  return 0;
}

// Defined with the allocation-free entry below: that entry's own status word, 0 when the entry
// has not been used on the device.
static int static_status_read_clear(int dev, unsigned int* value);

extern "C" int fastnn_b200_device_status(unsigned int* status) {
  int dev = -1;
  FNN_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return -1;
  FNN_CUDA_OK(cudaDeviceSynchronize());
  unsigned int v = 0;
  DeviceState* st = current_state();
  if (st != nullptr) {
    FNN_CUDA_OK(cudaMemcpy(&v, st->status, sizeof(v), cudaMemcpyDeviceToHost));
    if (v != 0) FNN_CUDA_OK(cudaMemset(st->status, 0, sizeof(v)));
  }
  // kernels of fastnn_b200_gemm_splitk_static report into a word of their own (that entry works
  // without fastnn_cuda_init): the first non-zero code of the two is returned, both are cleared
  unsigned int vs = 0;
  if (static_status_read_clear(dev, &vs) != 0) return -1;
  if (status) *status = v != 0 ? v : vs;
  return 0;
}

extern "C" int fastnn_b200_selftest_bounded_wait(unsigned int budget_us, unsigned int* waited_us) {
  DeviceState* st = current_state();
  if (st == nullptr) return -1;
  if (budget_us < 1 || budget_us > 100000) return -1;            // 1 us .. 0.1 s
  int dev = 0, khz = 0;
  FNN_CUDA_OK(cudaGetDevice(&dev));
  if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev) != cudaSuccess || khz <= 0) {
    (void)cudaGetLastError();
    khz = 2000000;
  }
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.status = st->status;
  p.spin_budget = static_cast<long long>(budget_us) * khz / 1000;   // ticks at the maximum clock
  unsigned int* out = nullptr;
  FNN_CUDA_OK(cudaMalloc(&out, 2 * sizeof(unsigned int)));
  int rc = -1;
  unsigned int host[2] = {0u, 0u};
  if (cudaMemset(out, 0, 2 * sizeof(unsigned int)) == cudaSuccess) {
    fnn::bounded_wait_selftest_kernel<<<1, 32>>>(p, fnn::kStatusSelfTest, out);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (cudaGetLastError() == cudaSuccess && cudaDeviceSynchronize() == cudaSuccess &&
        cudaMemcpy(host, out, sizeof(host), cudaMemcpyDeviceToHost) == cudaSuccess)
      rc = host[0] == 1u ? 0 : -1;        // the wait must have given up
  }
  (void)cudaGetLastError();
  (void)cudaFree(out);
  if (waited_us) *waited_us = static_cast<unsigned int>(1000ull * host[1] / static_cast<unsigned>(khz));
  return rc;
}

extern "C" int fastnn_b200_gemm_gather_mc_ex(int layout, const float* a, const float* b, float* c, int m,
                                             int n, int k, int batch, long long lda, long long ldb,
                                             long long ldc, long long stride_a, long long stride_b,
                                             long long stride_c, float alpha, const float* bias, int act,
                                             float* mc_c, void* stream) {
  if (mc_c == nullptr) return -1;
  GemmArgs g{layout, a, b, c, m, n, k, batch, lda, ldb, ldc, stride_a, stride_b, stride_c,
             alpha, 0.0f, bias, act, static_cast<cudaStream_t>(stream)};
  g.mc_c = mc_c;
  return gemm_dispatch(g);
}

extern "C" int fastnn_b200_gemm_gather_ex(int layout, const float* a, const float* b, float* c, int m,
                                          int n, int k, int batch, long long lda, long long ldb,
                                          long long ldc, long long stride_a, long long stride_b,
                                          long long stride_c, float alpha, const float* bias, int act,
                                          float* const* peer_c, int n_peers, void* stream) {
  if (n_peers < 0 || n_peers > fnn::kMaxPeers) return -1;
  if (n_peers > 0 && peer_c == nullptr) return -1;
  GemmArgs g{layout, a, b, c, m, n, k, batch, lda, ldb, ldc, stride_a, stride_b, stride_c,
             alpha, 0.0f, bias, act, static_cast<cudaStream_t>(stream)};
  g.peer_c = peer_c;
  g.n_peers = n_peers;
  return gemm_dispatch(g);
}

extern "C" unsigned long long fastnn_b200_launch_count(void) {
  return g_launches.load(std::memory_order_relaxed);
}

extern "C" const char* fastnn_b200_version(void) { return "fastnn_b200 0.1 (sm_100a)"; }

// ======================================================== allocation-free entry ===
//
// Split-K GEMM whose partial sums live in a fixed array inside the library image instead of
// a cudaMalloc'ed workspace.  See the declaration in the header for who needs this and why.

namespace {

constexpr size_t kStaticScratchFloats = 4u * 1024u * 1024u;     // 16 MiB per device
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];
static __device__ unsigned int g_static_status;

struct StaticState {
  bool ready = false;
  float* scratch = nullptr;        // device address of g_static_scratch on this device
  unsigned int* status = nullptr;  // device address of g_static_status on this device
  int num_sms = 0;
  long long spin_budget = 0;
};
StaticState g_static[kMaxDevices];

// Once per device, with that device current.  Resolves device addresses of the two symbols
// (their host-side names are not device pointers) and the driver's tensor-map encoder.
// Nothing here allocates device memory.
int static_setup(int dev, StaticState** out) {
  StaticState& st = g_static[dev];
  if (!st.ready) {
    int major = 0, sms = 0, khz = 0;
    FNN_CUDA_OK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) {
      std::fprintf(stderr, "fastnn_b200: device %d is not sm_100; no kernel image for it\n", dev);
      return -1;
    }
    FNN_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev) != cudaSuccess || khz <= 0) {
      (void)cudaGetLastError();
      khz = 2000000;
    }
    void* p = nullptr;
    FNN_CUDA_OK(cudaGetSymbolAddress(&p, g_static_scratch));
    st.scratch = static_cast<float*>(p);
    p = nullptr;
    FNN_CUDA_OK(cudaGetSymbolAddress(&p, g_static_status));
    st.status = static_cast<unsigned int*>(p);
    if (st.scratch == nullptr || st.status == nullptr) return -1;
    if (resolve_encoder() != 0) return -1;
    FNN_CUDA_OK(cudaFuncSetAttribute(fnn::gemm_tf32_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(kMaxDynSmem)));
    st.num_sms = sms;
    st.spin_budget = 2000ll * khz;
    st.ready = true;
  }
  *out = &st;
  return 0;
}

}  // namespace

// Reads and clears the status word of the allocation-free entry on device `dev` (current).  A
// plain copy from the symbol's address: nothing is allocated.  0 when the entry was never used.
static int static_status_read_clear(int dev, unsigned int* value) {
  *value = 0;
  std::lock_guard<std::mutex> lock(g_mutex);
  const StaticState& st = g_static[dev];
  if (!st.ready) return 0;
  unsigned int v = 0;
  FNN_CUDA_OK(cudaMemcpy(&v, st.status, sizeof(v), cudaMemcpyDeviceToHost));
  if (v != 0) FNN_CUDA_OK(cudaMemset(st.status, 0, sizeof(v)));
  *value = v;
  return 0;
}

extern "C" int fastnn_b200_gemm_splitk_static(int layout, const float* a, const float* b, float* c,
                                              int m, int n, int k, int split_k, void* stream) {
  if (layout < 0 || layout > 2 || m < 0 || n < 0 || k < 1 || split_k < 1) return -1;
  if (m == 0 || n == 0) return 0;
  if (a == nullptr || b == nullptr || c == nullptr) return -1;
  const long long lda = (layout == FASTNN_B200_TN) ? m : k;
  const long long ldb = (layout == FASTNN_B200_NT) ? k : n;
  // TMA addressing rules for the operands and the float4 reduce pass over C
  if (!aligned16(a) || !aligned16(b) || !aligned16(c) || (lda & 3) || (ldb & 3) || (n & 3)) {
    std::fprintf(stderr, "fastnn_b200_gemm_splitk_static: operands must be 16-byte aligned with "
                         "row lengths that are multiples of 4 floats\n");
    return -1;
  }
  const int num_kb = ceil_div(k, fnn::kBlockK);
  if (split_k > num_kb) split_k = num_kb;
  const int kbps = ceil_div(num_kb, split_k);
  split_k = ceil_div(num_kb, kbps);
  const unsigned long long need = 1ull * m * n * split_k;
  if (need > kStaticScratchFloats) {
    std::fprintf(stderr, "fastnn_b200_gemm_splitk_static: m*n*split_k = %llu floats exceeds the "
                         "built-in scratch of %zu floats (16 MiB); use fewer splits or the "
                         "allocating entry points\n", need, kStaticScratchFloats);
    return -2;
  }
  int dev = -1;
  FNN_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return -1;
  std::lock_guard<std::mutex> lock(g_mutex);
  StaticState* st = nullptr;
  if (static_setup(dev, &st) != 0) return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  const int block_n = n >= 128 ? 128 : ceil_div(n, 32) * 32;
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.m = m; p.n = n; p.k = k; p.batch = 1;
  p.block_n = block_n;
  p.num_stages = stages_for(block_n);
  p.tiles_m = ceil_div(m, fnn::kBlockM);
  p.tiles_n = ceil_div(n, block_n);
  p.num_kb = num_kb;
  p.num_kb1 = num_kb;
  p.split_k = split_k + 0;
  p.kb_per_split = kbps;
  const long long units = 1ll * p.tiles_m * p.tiles_n * split_k;
  if (units > 0x7fffffffll) return -1;
  p.total_units = static_cast<int>(units);
  p.a_mn_major = (layout == FASTNN_B200_TN) ? 1 : 0;
  p.b_mn_major = (layout == FASTNN_B200_NT) ? 0 : 1;
  p.alpha = 1.0f; p.beta = 0.0f; p.bias = nullptr; p.act = 0;
  p.status = st->status;
  p.spin_budget = st->spin_budget;
  p.store_mode = 0;
  p.group_m = fnn::kGroupM;
  p.c = st->scratch; p.ldc = n; p.c_batch_stride = 1ll * m * n;
  // With alpha = 1, beta = 0 and no bias the kernel's epilogue is the identity, so a single
  // split also lands in the scratch unchanged and the reduce pass copies it to C.

  CUtensorMap tmA, tmB, tmC;
  bool ok;
  if (!p.a_mn_major)
    ok = encode_map(&tmA, a, k, m, 1, lda * 4ull, lda * 4ull * m, fnn::kBlockK, fnn::kBlockM);
  else
    ok = encode_map(&tmA, a, m, k, 1, lda * 4ull, lda * 4ull * k, 32, fnn::kBlockK, true);
  if (!p.b_mn_major)
    ok = ok && encode_map(&tmB, b, k, n, 1, ldb * 4ull, ldb * 4ull * n, fnn::kBlockK, block_n);
  else
    ok = ok && encode_map(&tmB, b, n, k, 1, ldb * 4ull, ldb * 4ull * k, 32, fnn::kBlockK, true);
  ok = ok && encode_map(&tmC, st->scratch, n, m, static_cast<uint64_t>(split_k), n * 4ull,
                        4ull * m * n, 32, 32);
  if (!ok) return -1;
  const int grid = p.total_units < st->num_sms ? p.total_units : st->num_sms;
  fnn::gemm_tf32_kernel<<<grid, fnn::kNumThreads, fnn::gemm_smem_bytes(block_n, p.num_stages), s>>>(
      tmA, tmB, tmC, tmA, tmB, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  FNN_CUDA_OK(cudaGetLastError());
  long long blocks = (1ll * m * n / 4 + 255) / 256;
  if (blocks > 8ll * st->num_sms) blocks = 8ll * st->num_sms;
  if (blocks < 1) blocks = 1;
  fnn::splitk_reduce_vec4_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(
      reinterpret_cast<const float4*>(st->scratch), c, nullptr, m, n, 1, split_k, n,
      1ll * m * n, 1.0f, 0.0f, 0);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  FNN_CUDA_OK(cudaGetLastError());
  t_last = LastCall{2, block_n, split_k, grid};
  return 0;
}
