// C ABI over the kernels: plans (tensor maps, flags, status words) and launches.
// The harness this replaces is backend/node/run_tma.py:47-175 (encode the maps the header
// names, allocate and zero the kernel's own buffers once, launch with the cluster
// attribute) and backend/node/clusterlaunch.py:34-51.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "../../include/warpc_b200.h"
#include "gemm_kernel.cuh"
#include "kernel_table.h"

namespace {

using namespace wb;

// ------------------------------------------------------------------ kernel table
template <class C>
wb_kernel_entry entry(int id, const char* name) {
  wb_kernel_entry e;
  e.id = id, e.cg = C::CG, e.tile_m = C::TM, e.tile_n = C::TN, e.direct = C::DIRECT ? 1 : 0, e.simple = C::SIMPLE ? 1 : 0, e.ksub = C::KSUB, e.mode = C::MODE;
  e.reps = C::REPS, e.epi_rows = C::EPI_ROWS, e.wide_rows = C::WIDE_ROWS, e.ncols = C::NCOLS, e.stage_bytes = C::STAGE_BYTES;
  e.smem_fixed = C::smem_bytes(0);
  e.staging_bytes = C::STAGING_BYTES;
  e.name = name;
  e.fn = reinterpret_cast<const void*>(&gemm_kernel<C>);
  return e;
}

#define WB_KERNELS(X)                       \
  X(0, 1, 128, 128, true, "one_128x128_direct")      \
  X(1, 2, 128, 64, true, "pair_128x64_direct")       \
  X(2, 2, 128, 64, false, "pair_128x64_staged")      \
  X(3, 2, 128, 128, true, "pair_128x128_direct")     \
  X(4, 2, 128, 128, false, "pair_128x128_staged")    \
  X(5, 2, 192, 128, true, "pair_192x128_direct")     \
  X(6, 2, 192, 128, false, "pair_192x128_staged")    \
  X(7, 2, 256, 128, true, "pair_256x128_direct")     \
  X(8, 2, 256, 128, false, "pair_256x128_staged")    \
  X(9, 2, 256, 256, true, "pair_256x256_direct")     \
  X(10, 2, 256, 256, false, "pair_256x256_staged")   \
  X(11, 2, 256, 64, false, "pair_256x64_staged")     \
  X(12, 2, 128, 256, false, "pair_128x256_staged")

const wb_kernel_entry* table() {
  static wb_kernel_entry t[] = {
#define X(id, cg, tm, tn, direct, name) entry<Cfg<cg, tm, tn, direct>>(id, name),
      WB_KERNELS(X)
#undef X
      // whole tiles, one a CTA or by stride, stored from the registers, the ring's round fixed: a quarter of the code
      entry<Cfg<2, 128, 64, true, 32, 2, true, 4>>(13, "pair_128x64_simple"),
      entry<Cfg<2, 128, 128, true, 32, 2, true, 2>>(14, "pair_128x128_simple"),
      entry<Cfg<2, 256, 128, true, 32, 2, true, 1>>(15, "pair_256x128_simple"),
      // one scheduling mode each, for the three long programs the rule names: stream-K on 256 x 128 tiles, launch control
      // and split-K over the grid on 256 x 256 tiles (staged store; phase stamps and further copies of C as in the full ones)
      entry<Cfg<2, 256, 128, false, 32, 2, false, 0, SCHED_STREAMK>>(16, "pair_256x128_staged_stream_k"),
      entry<Cfg<2, 256, 256, false, 32, 2, false, 0, SCHED_CLC>>(17, "pair_256x256_staged_launch_control"),
      entry<Cfg<2, 256, 256, false, 32, 2, false, 0, SCHED_SPLITK>>(18, "pair_256x256_staged_split_k"),
  };
  return t;
}
constexpr int kKernels = 19;

// ------------------------------------------------------------------ driver entry points
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// A row-major rows x cols matrix, box = box_rows x box_cols, 128-byte swizzle (operands) or none
// (the C staging boxes), zero fill
// out of bounds -- the map backend/node/run_tma.py:32-45 encodes from a `.tmap` line.
int encode_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem, const void* ptr, int rows, int cols, int box_rows, int box_cols,
              CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B, int ld = 0) {
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return WG_E_NODRIVER;
  cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
  cuuint64_t strides[1] = {cuuint64_t(ld > 0 ? ld : cols) * cuuint64_t(elem)};  // ld: elements between rows, when the matrix is a block of a wider one
  cuuint32_t box[2] = {cuuint32_t(box_cols), cuuint32_t(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  // L2 promotion of the maps' loads: 128 bytes as the reference's harness encodes them, WARPC_L2PROMO=0..3 to try
  // another (none, 64, 128, 256 bytes: backend/node/run_tma.py:42)
  int promo = int(CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
  if (const char* e = std::getenv("WARPC_L2PROMO"))
    if (e[0] >= '0' && e[0] <= '3' && e[1] == 0) promo = e[0] - '0';
  CUresult r = enc(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle, CUtensorMapL2promotion(promo), CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? WG_OK : int(r);
}

// L2 hints, from measurements on the benchmark shapes (isolated calls on L2-warm operands): operand
// lines marked evict-last pay where every CTA has one tile or the tiles' K is short and A and B^T
// together are well inside the L2 (2048^3 -8 %, 3072x1280x2048 -9 %, 4096x4096x1024 -5 %) and cost
// where they are not (8192x2048x4096 +6 %); C marked evict-first pays on the persistent walks, whose
// stores run beside the next tile's loads (4096^3 -2 %, 2048x2048x16384 -2 %), and never costs.
int l2_hints_for(const wg_launch_info& li, int M, int N, int K) {
  const bool small_operands = 2.0 * double(K) * (double(M) + double(N)) <= 48.0 * 1024 * 1024;
  const bool loads_last = (li.sched == SCHED_ONE || li.sched == SCHED_STRIDE) && small_operands;
  const bool stores_first = li.sched == SCHED_STRIDE || li.sched == SCHED_STREAMK || loads_last;
  return (stores_first ? 1 : 0) | (loads_last ? 2 : 0);
}

struct Plan {
  int device = 0;
  wg_variant v;
  wg_launch_info li;
  const wb_kernel_entry* k = nullptr;
  CUtensorMap map_a, map_b, map_c, map_cw;
  KParams p;
  uint32_t* d_flags = nullptr;
  uint32_t* d_status = nullptr;
  float* d_ws = nullptr;
  CUtensorMap* d_replicas = nullptr;
  int ldc = 0;
  unsigned long long* d_stamps = nullptr;
  size_t flag_bytes = 0;
  // host plans own these
  void *dA = nullptr, *dBt = nullptr, *dC = nullptr;
  bool owns_buffers = false;
  bool dependent_launch = false;
  // host plans of large problems: the product as a grid of blocks, each with a plan of its own, so that the copies in,
  // the launches and the copies out run as a pipeline (see wg_host_run)
  std::vector<Plan*> blocks;
  int block_rows = 0, block_cols = 0;
  cudaStream_t s_in = nullptr, s_mm = nullptr, s_out = nullptr;
  std::vector<cudaEvent_t> ev_a, ev_b, ev_mm;  // launches carry the programmatic stream serialization attribute
  int M = 0, N = 0, K = 0;
};

#define WG_CUDA(call)                          \
  do {                                         \
    cudaError_t e_ = (call);                   \
    if (e_ != cudaSuccess) return int(e_);     \
  } while (0)

// Makes `device` current for the length of an entry point and gives the caller's device back on
// the way out, so one host thread can drive plans on several GPUs in turn.
struct DeviceGuard {
  int prev = -1;
  bool changed = false;
  cudaError_t err = cudaSuccess;
  explicit DeviceGuard(int device) {
    err = cudaGetDevice(&prev);
    if (err == cudaSuccess && prev != device) {
      err = cudaSetDevice(device);
      changed = err == cudaSuccess;
    }
  }
  ~DeviceGuard() {
    if (changed) cudaSetDevice(prev);
  }
  DeviceGuard(const DeviceGuard&) = delete;
  DeviceGuard& operator=(const DeviceGuard&) = delete;
};
#define WG_ON_DEVICE(device)        \
  DeviceGuard guard_(device);       \
  if (guard_.err != cudaSuccess) return int(guard_.err)

void launch_config(const wg_launch_info& li, cudaStream_t stream, bool dependent, cudaLaunchConfig_t* cfg, cudaLaunchAttribute attr[2]) {
  std::memset(cfg, 0, sizeof *cfg);
  cfg->gridDim = dim3(unsigned(li.grid), 1, 1);
  cfg->blockDim = dim3(unsigned(li.threads), 1, 1);
  cfg->dynamicSmemBytes = size_t(li.dynsmem);
  cfg->stream = stream;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = unsigned(li.cluster);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg->attrs = attr;
  cfg->numAttrs = dependent ? 2 : 1;
}

// The attribute is per kernel function, not per launch, and plans with rings of different depth share a function: it is
// always raised to the most a CTA may have, so a plan made later never lowers it under a plan made earlier.
constexpr int kMaxDynSmem = 232448;

// Split-K and stream-K CTAs wait for each other's flags, so every cluster of the grid has to be
// resident at once.  The rule's tables assume a whole B200 (148 SMs, 74 resident pairs); a device
// or context that offers fewer is refused here rather than found out by a wait that runs out.
int check_coresident(const wb_kernel_entry* k, const wg_launch_info& li) {
  if (li.sched != SCHED_SPLITK && li.sched != SCHED_STREAMK) return WG_OK;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  launch_config(li, nullptr, false, &cfg, attr);
  WG_CUDA(cudaFuncSetAttribute(k->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem));
  int clusters = 0;
  WG_CUDA(cudaOccupancyMaxActiveClusters(&clusters, k->fn, &cfg));
  return li.grid / li.cluster <= clusters ? WG_OK : WG_E_VARIANT;
}

int fill_plan(Plan* pl, int device, const wg_variant* v, int M, int N, int K, const void* dA, const void* dBt, void* dC, int ldc = 0) {
  if (!v || !dA || !dBt || !dC) return WG_E_ARG;
  if ((reinterpret_cast<uintptr_t>(dA) | reinterpret_cast<uintptr_t>(dBt) | reinterpret_cast<uintptr_t>(dC)) & 15u) return WG_E_ARG;
  if (M <= 0 || N <= 0 || K <= 0 || K % 64 != 0 || N % 4 != 0) return WG_E_ARG;
  pl->device = device, pl->v = *v, pl->M = M, pl->N = N, pl->K = K;
  int r = wg_realise(v, M, N, K, &pl->li);
  if (r != WG_OK) return r;
  const wg_launch_info& li = pl->li;
  pl->k = wb_kernel_at(li.kernel_id);
  WG_ON_DEVICE(device);
  std::memset(&pl->map_c, 0, sizeof pl->map_c);
  std::memset(&pl->map_cw, 0, sizeof pl->map_cw);
  if ((r = encode_2d(&pl->map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, dA, M, K, li.a_box_rows, 64)) != WG_OK) return r;
  if ((r = encode_2d(&pl->map_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, dBt, N, K, li.bt_box_rows, 64)) != WG_OK) return r;
  if (!li.direct && (r = encode_2d(&pl->map_c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dC, M, N, li.c_box_rows, 32, CU_TENSOR_MAP_SWIZZLE_NONE, ldc)) != WG_OK) return r;
  if (!li.direct && (r = encode_2d(&pl->map_cw, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dC, M, N, pl->k->wide_rows, 32, CU_TENSOR_MAP_SWIZZLE_NONE, ldc)) != WG_OK) return r;
  pl->flag_bytes = size_t(li.nflags > 0 ? li.nflags : 1) * sizeof(uint32_t);
  WG_CUDA(cudaMalloc(&pl->d_flags, pl->flag_bytes));
  WG_CUDA(cudaMalloc(&pl->d_status, 8 * sizeof(uint32_t)));
  if (li.ws_words > 0) WG_CUDA(cudaMalloc(&pl->d_ws, size_t(li.ws_words) * sizeof(float)));  // every word is written before it is read
  WG_CUDA(cudaMemsetAsync(pl->d_flags, 0, pl->flag_bytes, 0));
  WG_CUDA(cudaMemsetAsync(pl->d_status, 0, 8 * sizeof(uint32_t), 0));
  WG_CUDA(cudaStreamSynchronize(0));  // the words are zero before any stream, blocking or not, can launch on the plan
  KParams& p = pl->p;
  std::memset(&p, 0, sizeof p);
  p.M = M, p.N = N, p.K = K;
  pl->ldc = ldc;
  p.ldc = ldc > 0 ? ldc : N;
  p.kt = K / 64;
  const int tiles_m = (M + li.tile_m - 1) / li.tile_m, tiles_n = (N + li.tile_n - 1) / li.tile_n;
  p.ntiles = tiles_m * tiles_n;
  p.cl_n = li.cl_n > 0 ? li.cl_n : 1;
  p.group = li.group > 0 ? li.group : 1;
  p.serp = li.serpentine;
  p.depth = li.depth, p.nbuf = li.nbuf, p.sched = li.sched, p.ask_ahead = li.ask_ahead;
  p.split = li.split;
  p.ksub = li.ksub, p.rounds = li.rounds;
  p.l2_hints = l2_hints_for(li, M, N, K);
  p.staging_bytes = li.staging_bytes;
  p.late_launch = v->late_launch;
  p.epi_ring = li.wide_rows != 0;
  if (li.sched == SCHED_STREAMK) {
    const int clusters = li.grid / li.cluster, units = (p.ntiles / li.cluster - li.sk_dp) * p.kt;
    p.sk_clusters = clusters, p.sk_q = units / clusters, p.sk_r = units % clusters, p.sk_dp = li.sk_dp;
  }
  p.C = static_cast<float*>(dC);
  p.flags = pl->d_flags;
  p.ws = pl->d_ws;
  p.status = pl->d_status;
  p.timeout_ns = 2000ull * 1000ull * 1000ull;
  WG_CUDA(cudaFuncSetAttribute(pl->k->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem));
  return check_coresident(pl->k, li);
}

// A host plan of a large problem runs as a pipeline: C is cut into blocks of 2048 x 2048, block (i, j) = rows i of A
// times rows j of B^T, each with the rule's own program for a 2048 x 2048 x K product.  The row panels of A and B^T
// go to the device alternately (A0, B0, A1, B1, ...); a block is launched when its two panels have landed and copied
// out when it is done, so the copies in, the tensor cores and the copies out overlap instead of following each other.
// Only for problems that cut evenly and are worth it (>= 256 MB moved); otherwise one shot with the plan's own
// variant.  (The variant a host plan was made with names the one-shot program; the blocks run the rule's.)
int make_blocks(Plan* pl, int device) {
  constexpr int B = 2048;
  const int M = pl->M, N = pl->N, K = pl->K;
  const double moved = 2.0 * K * (double(M) + N) + 4.0 * M * N;
  if (M % B != 0 || N % B != 0 || M / B * (N / B) < 4 || M / B * (N / B) > 1024 || moved < 256e6) return WG_OK;
  wg_variant bv;
  if (wg_choose(B, B, K, WG_SM_100A, &bv) != WG_OK) return WG_OK;
  const int nr = M / B, nc = N / B;
  for (int i = 0; i < nr; ++i)
    for (int j = 0; j < nc; ++j) {
      Plan* b = new (std::nothrow) Plan();
      if (!b) return WG_E_ARG;
      pl->blocks.push_back(b);
      const int r = fill_plan(b, device, &bv, B, B, K, static_cast<const char*>(pl->dA) + size_t(i) * B * K * 2,
                              static_cast<const char*>(pl->dBt) + size_t(j) * B * K * 2,
                              static_cast<char*>(pl->dC) + (size_t(i) * B * N + size_t(j) * B) * 4, N);
      if (r != WG_OK) return r;
    }
  pl->block_rows = nr, pl->block_cols = nc;
  WG_CUDA(cudaStreamCreateWithFlags(&pl->s_in, cudaStreamNonBlocking));
  WG_CUDA(cudaStreamCreateWithFlags(&pl->s_mm, cudaStreamNonBlocking));
  WG_CUDA(cudaStreamCreateWithFlags(&pl->s_out, cudaStreamNonBlocking));
  pl->ev_a.resize(nr), pl->ev_b.resize(nc), pl->ev_mm.resize(size_t(nr) * nc);
  for (auto* list : {&pl->ev_a, &pl->ev_b, &pl->ev_mm})
    for (auto& e : *list) WG_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  return WG_OK;
}

// The pipelined form of wg_host_run (see make_blocks).  Panels go in on one stream in the order A0 B0 A1 B1 ...;
// block (i, j) waits for panels i and j on the compute stream, blocks are launched in the order their panels
// complete (all blocks with max(i, j) = d after panel pair d), and each goes out on a third stream once computed.
int host_run_blocks(Plan* pl, const void* hA, const void* hBt, void* hC) {
  constexpr int B = 2048;
  const int nr = pl->block_rows, nc = pl->block_cols, N = pl->N, K = pl->K;
  const size_t panel = size_t(B) * K * 2;
  for (int d = 0; d < (nr > nc ? nr : nc); ++d) {
    if (d < nr) {
      WG_CUDA(cudaMemcpyAsync(static_cast<char*>(pl->dA) + d * panel, static_cast<const char*>(hA) + d * panel, panel, cudaMemcpyHostToDevice, pl->s_in));
      WG_CUDA(cudaEventRecord(pl->ev_a[d], pl->s_in));
    }
    if (d < nc) {
      WG_CUDA(cudaMemcpyAsync(static_cast<char*>(pl->dBt) + d * panel, static_cast<const char*>(hBt) + d * panel, panel, cudaMemcpyHostToDevice, pl->s_in));
      WG_CUDA(cudaEventRecord(pl->ev_b[d], pl->s_in));
    }
    auto run_block = [&](int i, int j) -> int {
      WG_CUDA(cudaStreamWaitEvent(pl->s_mm, pl->ev_a[i], 0));
      WG_CUDA(cudaStreamWaitEvent(pl->s_mm, pl->ev_b[j], 0));
      return wg_launch(pl->blocks[size_t(i) * nc + j], pl->s_mm);
    };
    // rows [r0, r0 + rows) x columns [c0, c0 + cols) of C out, once everything launched so far is done
    auto copy_out = [&](cudaEvent_t done, int r0, int rows, int c0, int cols) -> int {
      WG_CUDA(cudaEventRecord(done, pl->s_mm));
      WG_CUDA(cudaStreamWaitEvent(pl->s_out, done, 0));
      const size_t off = (size_t(r0) * N + size_t(c0)) * 4;
      WG_CUDA(cudaMemcpy2DAsync(static_cast<char*>(hC) + off, size_t(N) * 4, static_cast<const char*>(pl->dC) + off, size_t(N) * 4, size_t(cols) * 4,
                                size_t(rows), cudaMemcpyDeviceToHost, pl->s_out));
      return WG_OK;
    };
    int r = WG_OK;
    // the new row of blocks (d, 0..d) leaves as one copy of long rows, the new column (0..d-1, d) as one of many rows
    if (d < nr) {
      const int last = d < nc ? d : nc - 1;
      for (int j = 0; j <= last && r == WG_OK; ++j) r = run_block(d, j);
      if (r == WG_OK) r = copy_out(pl->ev_mm[size_t(d) * nc], d * B, B, 0, (last + 1) * B);
    }
    if (d < nc && d > 0 && r == WG_OK) {
      const int rows = d < nr ? d : nr;
      for (int i = 0; i < rows && r == WG_OK; ++i) r = run_block(i, d);
      if (r == WG_OK) r = copy_out(pl->ev_mm[size_t(0) * nc + d], 0, rows * B, d * B, B);
    }
    if (r != WG_OK) return r;
  }
  WG_CUDA(cudaStreamSynchronize(pl->s_out));
  WG_CUDA(cudaStreamSynchronize(pl->s_mm));
  return WG_OK;
}

}  // namespace

const wb_kernel_entry* wb_find_kernel(int cg, int tile_m, int tile_n, int direct, int simple, int mode) {
  const wb_kernel_entry* t = table();
  for (int i = 0; i < kKernels; ++i)
    if (t[i].cg == cg && t[i].tile_m == tile_m && t[i].tile_n == tile_n && t[i].direct == direct && t[i].simple == simple && t[i].mode == mode)
      return &t[i];
  return nullptr;
}
const wb_kernel_entry* wb_kernel_at(int id) { return (id >= 0 && id < kKernels) ? &table()[id] : nullptr; }
int wb_kernel_total() { return kKernels; }

extern "C" int wg_kernel_count(void) { return kKernels; }
extern "C" const char* wg_kernel_name(int id) {
  const wb_kernel_entry* e = wb_kernel_at(id);
  return e ? e->name : "?";
}

extern "C" int wg_plan_create(int device, const wg_variant* v, int M, int N, int K, const void* dA, const void* dBt, void* dC,
                              void** plan) {
  if (!plan) return WG_E_ARG;
  *plan = nullptr;
  Plan* pl = new (std::nothrow) Plan();
  if (!pl) return WG_E_ARG;
  const int r = fill_plan(pl, device, v, M, N, K, dA, dBt, dC);
  if (r != WG_OK) {
    wg_plan_destroy(pl);
    return r;
  }
  *plan = pl;
  return WG_OK;
}

extern "C" int wg_plan_create_block(int device, const wg_variant* v, int M, int N, int K, const void* dA, const void* dBt, void* dC, int ldc,
                                    void** plan) {
  if (!plan || ldc < N || ldc % 4 != 0) return WG_E_ARG;
  *plan = nullptr;
  Plan* pl = new (std::nothrow) Plan();
  if (!pl) return WG_E_ARG;
  const int r = fill_plan(pl, device, v, M, N, K, dA, dBt, dC, ldc);
  if (r != WG_OK) {
    wg_plan_destroy(pl);
    return r;
  }
  *plan = pl;
  return WG_OK;
}

extern "C" int wg_host_plan_create(int device, const wg_variant* v, int M, int N, int K, void** plan) {
  if (!plan || !v || M <= 0 || N <= 0 || K <= 0) return WG_E_ARG;
  *plan = nullptr;
  Plan* pl = new (std::nothrow) Plan();
  if (!pl) return WG_E_ARG;
  pl->owns_buffers = true;
  pl->device = device;
  DeviceGuard guard(device);
  int r = int(guard.err);
  if (r == 0) r = int(cudaMalloc(&pl->dA, size_t(M) * K * 2));
  if (r == 0) r = int(cudaMalloc(&pl->dBt, size_t(N) * K * 2));
  if (r == 0) r = int(cudaMalloc(&pl->dC, size_t(M) * N * 4));
  if (r == 0) r = fill_plan(pl, device, v, M, N, K, pl->dA, pl->dBt, pl->dC);
  if (r == 0) r = make_blocks(pl, device);
  if (r != WG_OK) {
    wg_plan_destroy(pl);
    return r;
  }
  *plan = pl;
  return WG_OK;
}

extern "C" void* wg_host_plan_buffer(void* plan, int which) {
  Plan* pl = static_cast<Plan*>(plan);
  if (!pl) return nullptr;
  return which == 0 ? pl->dA : which == 1 ? pl->dBt : which == 2 ? pl->dC : nullptr;
}

extern "C" int wg_plan_set_timeout_ms(void* plan, unsigned ms) {
  Plan* pl = static_cast<Plan*>(plan);
  if (!pl) return WG_E_ARG;
  pl->p.timeout_ns = (ms ? ms : 2000u) * 1000000ull;
  return WG_OK;
}

extern "C" int wg_plan_info(void* plan, wg_launch_info* out) {
  Plan* pl = static_cast<Plan*>(plan);
  if (!pl || !out) return WG_E_ARG;
  *out = pl->li;
  return WG_OK;
}

extern "C" int wg_launch(void* plan, void* cuda_stream) {
  Plan* pl = static_cast<Plan*>(plan);
  if (!pl || !pl->k) return WG_E_ARG;
  WG_ON_DEVICE(pl->device);
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  launch_config(pl->li, static_cast<cudaStream_t>(cuda_stream), pl->dependent_launch, &cfg, attr);
  void* args[5] = {&pl->map_a, &pl->map_b, &pl->map_c, &pl->map_cw, &pl->p};
  // a simple instance takes no phase stamps: a plan asked for them launches the full instance of the same tile and store
  const wb_kernel_entry* k = pl->k;
  if (k->simple && pl->p.stamps != nullptr && !kSimpleStamps) {
    k = wb_find_kernel(k->cg, k->tile_m, k->tile_n, k->direct, 0, -1);
    if (!k) return WG_E_NOKERNEL;
    WG_CUDA(cudaFuncSetAttribute(k->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem));
  }
  return int(cudaLaunchKernelExC(&cfg, k->fn, args));
}

extern "C" int wg_plan_set_replicas(void* plan, int n, void* const* peer_dC) {
  Plan* pl = static_cast<Plan*>(plan);
  if (!pl || n < 0 || n > 15 || (n > 0 && !peer_dC)) return WG_E_ARG;
  WG_ON_DEVICE(pl->device);
  WG_CUDA(cudaDeviceSynchronize());  // no launch in flight reads the maps about to be replaced
  if (pl->d_replicas) cudaFree(pl->d_replicas);
  pl->d_replicas = nullptr, pl->p.replicas = nullptr, pl->p.rep_ptrs = nullptr, pl->p.nrep = 0;
  if (n == 0) return WG_OK;
  const wg_launch_info& li = pl->li;
  if (li.direct || li.sched == SCHED_SPLITK || li.sched == SCHED_STREAMK) return WG_E_VARIANT;
  if (pl->M % li.tile_m != 0 || pl->N % li.tile_n != 0) return WG_E_VARIANT;  // whole tiles only: the forwarding warp copies without bounds
  std::vector<CUtensorMap> maps(size_t(2 * n));
  for (int r = 0; r < n; ++r) {
    if (!peer_dC[r] || (reinterpret_cast<uintptr_t>(peer_dC[r]) & 15u)) return WG_E_ARG;
    int e = encode_2d(&maps[size_t(2 * r)], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, peer_dC[r], pl->M, pl->N, li.c_box_rows, 32, CU_TENSOR_MAP_SWIZZLE_NONE, pl->ldc);
    if (e == WG_OK)
      e = encode_2d(&maps[size_t(2 * r + 1)], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, peer_dC[r], pl->M, pl->N, pl->k->wide_rows, 32, CU_TENSOR_MAP_SWIZZLE_NONE, pl->ldc);
    if (e != WG_OK) return e;
  }
  // the maps, then the same copies' plain addresses, in one allocation
  const size_t map_bytes = maps.size() * sizeof(CUtensorMap);
  WG_CUDA(cudaMalloc(&pl->d_replicas, map_bytes + size_t(n) * sizeof(float*)));
  WG_CUDA(cudaMemcpy(pl->d_replicas, maps.data(), map_bytes, cudaMemcpyHostToDevice));
  WG_CUDA(cudaMemcpy(reinterpret_cast<char*>(pl->d_replicas) + map_bytes, peer_dC, size_t(n) * sizeof(float*), cudaMemcpyHostToDevice));
  pl->p.replicas = pl->d_replicas;
  pl->p.rep_ptrs = reinterpret_cast<float* const*>(reinterpret_cast<char*>(pl->d_replicas) + map_bytes);
  pl->p.nrep = n;
  return WG_OK;
}

// ------------------------------------------------------------------ buffers shared between processes (CUDA IPC)
namespace {
struct Imported {
  unsigned char handle[64];
  int device;
  void* base;
  int refs;
};
std::vector<Imported> g_imported;
std::mutex g_imported_mutex;
typedef CUresult (*AddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
}  // namespace

extern "C" int wg_ipc_export(int device, const void* dptr, unsigned char handle[64], unsigned long long* offset) {
  if (!dptr || !handle || !offset) return WG_E_ARG;
  WG_ON_DEVICE(device);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return WG_E_NODRIVER;
  CUdeviceptr base = 0;
  size_t size = 0;
  const CUresult r = reinterpret_cast<AddressRangeFn>(fn)(&base, &size, reinterpret_cast<CUdeviceptr>(dptr));
  if (r != CUDA_SUCCESS) return int(r);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
  cudaIpcMemHandle_t h;
  WG_CUDA(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
  std::memcpy(handle, &h, 64);
  *offset = reinterpret_cast<CUdeviceptr>(dptr) - base;
  return WG_OK;
}

extern "C" int wg_ipc_import(int device, const unsigned char handle[64], unsigned long long offset, void** dptr) {
  if (!handle || !dptr) return WG_E_ARG;
  *dptr = nullptr;
  WG_ON_DEVICE(device);  // the importing GPU is current: the mapping (and its peer access) is made for this device
  std::lock_guard<std::mutex> lock(g_imported_mutex);
  for (Imported& im : g_imported)
    if (im.device == device && std::memcmp(im.handle, handle, 64) == 0) {
      im.refs += 1;
      *dptr = static_cast<char*>(im.base) + offset;
      return WG_OK;
    }
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  void* base = nullptr;
  WG_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
  Imported im;
  std::memcpy(im.handle, handle, 64);
  im.device = device, im.base = base, im.refs = 1;
  g_imported.push_back(im);
  *dptr = static_cast<char*>(base) + offset;
  return WG_OK;
}

extern "C" int wg_ipc_release(int device, void* dptr) {
  if (!dptr) return WG_E_ARG;
  WG_ON_DEVICE(device);
  std::lock_guard<std::mutex> lock(g_imported_mutex);
  // the mapping whose base is the closest at or below the pointer
  int best = -1;
  for (size_t i = 0; i < g_imported.size(); ++i)
    if (g_imported[i].device == device && g_imported[i].base <= dptr &&
        (best < 0 || g_imported[i].base > g_imported[size_t(best)].base)) best = int(i);
  if (best < 0) return WG_E_ARG;
  if (--g_imported[size_t(best)].refs == 0) {
    const cudaError_t e = cudaIpcCloseMemHandle(g_imported[size_t(best)].base);
    g_imported.erase(g_imported.begin() + best);
    if (e != cudaSuccess) return int(e);
  }
  return WG_OK;
}

extern "C" int wg_plan_set_dependent_launch(void* plan, int on) {
  Plan* pl = static_cast<Plan*>(plan);
  if (!pl) return WG_E_ARG;
  pl->dependent_launch = on != 0;
  return WG_OK;
}

extern "C" int wg_last_device_status(void* plan, unsigned out[4]) {
  Plan* pl = static_cast<Plan*>(plan);
  if (!pl || !out) return WG_E_ARG;
  WG_ON_DEVICE(pl->device);
  uint32_t st[8];
  WG_CUDA(cudaDeviceSynchronize());
  WG_CUDA(cudaMemcpy(st, pl->d_status, sizeof st, cudaMemcpyDeviceToHost));
  for (int i = 0; i < 4; ++i) out[i] = st[i];
  return st[0] == 0 ? WG_OK : WG_E_DEVICE_WAIT;
}

extern "C" int wg_plan_reset(void* plan) {
  Plan* pl = static_cast<Plan*>(plan);
  if (!pl) return WG_E_ARG;
  WG_ON_DEVICE(pl->device);
  WG_CUDA(cudaDeviceSynchronize());
  WG_CUDA(cudaMemsetAsync(pl->d_flags, 0, pl->flag_bytes, 0));
  WG_CUDA(cudaMemsetAsync(pl->d_status, 0, 8 * sizeof(uint32_t), 0));
  WG_CUDA(cudaStreamSynchronize(0));
  return WG_OK;
}

extern "C" int wg_plan_destroy(void* plan) {
  Plan* pl = static_cast<Plan*>(plan);
  if (!pl) return WG_OK;
  DeviceGuard guard(pl->device);
  if (pl->d_flags) cudaFree(pl->d_flags);
  if (pl->d_status) cudaFree(pl->d_status);
  if (pl->d_ws) cudaFree(pl->d_ws);
  if (pl->d_replicas) cudaFree(pl->d_replicas);
  if (pl->d_stamps) cudaFree(pl->d_stamps);
  for (Plan* b : pl->blocks) wg_plan_destroy(b);
  for (auto* list : {&pl->ev_a, &pl->ev_b, &pl->ev_mm})
    for (auto& e : *list)
      if (e) cudaEventDestroy(e);
  for (cudaStream_t s : {pl->s_in, pl->s_mm, pl->s_out})
    if (s) cudaStreamDestroy(s);
  if (pl->owns_buffers) {
    if (pl->dA) cudaFree(pl->dA);
    if (pl->dBt) cudaFree(pl->dBt);
    if (pl->dC) cudaFree(pl->dC);
  }
  delete pl;
  return WG_OK;
}

extern "C" int wg_host_run(void* plan, const void* hA, const void* hBt, void* hC) {
  Plan* pl = static_cast<Plan*>(plan);
  if (!pl || !pl->owns_buffers || !hA || !hBt || !hC) return WG_E_ARG;
  WG_ON_DEVICE(pl->device);
  if (!pl->blocks.empty()) return host_run_blocks(pl, hA, hBt, hC);
  WG_CUDA(cudaMemcpyAsync(pl->dA, hA, size_t(pl->M) * pl->K * 2, cudaMemcpyHostToDevice, 0));
  WG_CUDA(cudaMemcpyAsync(pl->dBt, hBt, size_t(pl->N) * pl->K * 2, cudaMemcpyHostToDevice, 0));
  const int r = wg_launch(pl, nullptr);
  if (r != WG_OK) return r;
  WG_CUDA(cudaMemcpyAsync(hC, pl->dC, size_t(pl->M) * pl->N * 4, cudaMemcpyDeviceToHost, 0));
  WG_CUDA(cudaStreamSynchronize(0));
  return WG_OK;
}

// Mean milliseconds of `repeat` launches back to back between two CUDA events on the default
// stream, after `warmup` untimed ones -- the timing backend/node/run_tma.py:171-175 takes.
extern "C" int wg_time_launches(void* plan, int warmup, int repeat, float* ms_mean) {
  Plan* pl = static_cast<Plan*>(plan);
  if (!pl || !ms_mean || repeat < 1) return WG_E_ARG;
  WG_ON_DEVICE(pl->device);
  cudaEvent_t e0, e1;
  WG_CUDA(cudaEventCreate(&e0));
  WG_CUDA(cudaEventCreate(&e1));
  int r = WG_OK;
  for (int i = 0; i < warmup && r == WG_OK; ++i) r = wg_launch(pl, nullptr);
  if (r == WG_OK) r = int(cudaEventRecord(e0, 0));
  for (int i = 0; i < repeat && r == WG_OK; ++i) r = wg_launch(pl, nullptr);
  if (r == WG_OK) r = int(cudaEventRecord(e1, 0));
  if (r == WG_OK) r = int(cudaEventSynchronize(e1));
  float ms = 0;
  if (r == WG_OK) r = int(cudaEventElapsedTime(&ms, e0, e1));
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  *ms_mean = ms / float(repeat);
  return r;
}

// Timing runs: phase stamps (per CTA 64 events x 4 tiles, times on the GPU nanosecond timer or cycle sums) of the
// launches that follow; wg_plan_read_stamps synchronises and copies grid*256 words out.
extern "C" int wg_plan_enable_stamps(void* plan, int on) {
  Plan* pl = static_cast<Plan*>(plan);
  if (!pl) return WG_E_ARG;
  WG_ON_DEVICE(pl->device);
  const size_t bytes = size_t(pl->li.grid) * 256 * sizeof(unsigned long long);
  if (on && !pl->d_stamps) {
    WG_CUDA(cudaMalloc(&pl->d_stamps, bytes));
  }
  if (on) WG_CUDA(cudaMemset(pl->d_stamps, 0, bytes));
  pl->p.stamps = on ? pl->d_stamps : nullptr;
  return WG_OK;
}

extern "C" int wg_plan_read_stamps(void* plan, unsigned long long* out, size_t cap_words) {
  Plan* pl = static_cast<Plan*>(plan);
  if (!pl || !out || !pl->d_stamps) return WG_E_ARG;
  const size_t words = size_t(pl->li.grid) * 256;
  if (cap_words < words) return WG_E_ARG;
  WG_ON_DEVICE(pl->device);
  WG_CUDA(cudaDeviceSynchronize());
  WG_CUDA(cudaMemcpy(out, pl->d_stamps, words * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
  return int(words);
}

extern "C" int wg_tile_origin(const wg_launch_info* li, int tile, int* row, int* col) {
  if (!li || !row || !col || tile < 0) return WG_E_ARG;
  wb_tile_origin(tile, li->cg, li->tile_m, li->tile_n, li->group > 0 ? li->group : 1, li->cl_n > 0 ? li->cl_n : 1, li->serpentine, row, col);
  return WG_OK;
}

// Test hook for the bounded waits: overwrite one hand-off word of a split-K / stream-K plan.
// A CTA whose word disagrees with its partners' makes their flag waits run out, which must end
// as a recorded status (WG_E_DEVICE_WAIT), never as a hang.
extern "C" int wg_plan_debug_set_flag(void* plan, int index, unsigned value) {
  Plan* pl = static_cast<Plan*>(plan);
  if (!pl || index < 0 || size_t(index) * sizeof(uint32_t) >= pl->flag_bytes) return WG_E_ARG;
  WG_ON_DEVICE(pl->device);
  WG_CUDA(cudaDeviceSynchronize());
  WG_CUDA(cudaMemcpy(pl->d_flags + index, &value, sizeof value, cudaMemcpyHostToDevice));
  return WG_OK;
}

// ------------------------------------------------------------------ launch without allocating
// Some callers must not allocate device memory at the point of the call: code running inside
// another framework's memory pool or under a fixed memory budget, a real-time loop where
// cudaMalloc's implicit synchronisation is not acceptable, a library initialised after the
// application has handed all free memory to its own allocator.  For them the kernel's own
// words -- the split-K / stream-K hand-off flags and the status words -- live in one
// file-scope device array that every GPU loading this library holds until exit
// (WG_NOALLOC_MAX_FLAGS + 8 words = 16 KiB + 32 B).  Tensor maps travel as kernel parameters,
// so nothing else is needed.
constexpr int kNoAllocMaxFlags = 4096;
static __device__ __align__(256) uint32_t g_noalloc_scratch[kNoAllocMaxFlags + 8];

namespace {
constexpr int kMaxDevices = 64;
uint32_t* g_noalloc_ptr[kMaxDevices];  // device address of g_noalloc_scratch per device, 0 until set up
std::mutex g_noalloc_mutex;

// Once per device, with that device current: the array's name is only a host-side stand-in,
// the kernel needs the address the runtime reports for it.
int noalloc_setup(int device, uint32_t** out) {
  if (device < 0 || device >= kMaxDevices) return WG_E_ARG;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ptr[device]) {
    WG_ON_DEVICE(device);
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return int(e);
    if (!p) return WG_E_NODRIVER;
    g_noalloc_ptr[device] = static_cast<uint32_t*>(p);
  }
  *out = g_noalloc_ptr[device];
  return WG_OK;
}
}  // namespace

extern "C" int wg_noalloc_max_flags(void) { return kNoAllocMaxFlags; }

extern "C" int wg_launch_noalloc(int device, const wg_variant* v, int M, int N, int K, const void* dA, const void* dBt, void* dC,
                                 void* cuda_stream) {
  if (!dA || !dBt || !dC) return WG_E_ARG;
  if ((reinterpret_cast<uintptr_t>(dA) | reinterpret_cast<uintptr_t>(dBt) | reinterpret_cast<uintptr_t>(dC)) & 15u) return WG_E_ARG;
  if (M <= 0 || N <= 0 || K <= 0 || K % 64 != 0 || N % 4 != 0) return WG_E_ARG;
  wg_variant chosen;
  if (!v) {
    const int r = wg_choose(M, N, K, WG_SM_100A, &chosen);
    if (r != WG_OK) return r;
    v = &chosen;
  }
  wg_launch_info li;
  int r = wg_realise(v, M, N, K, &li);
  if (r != WG_OK) return r;
  if (li.nflags > kNoAllocMaxFlags || li.ws_words > 0) return WG_E_LIMIT;  // more hand-off words than the array holds, or a workspace
  uint32_t* scratch = nullptr;
  if ((r = noalloc_setup(device, &scratch)) != WG_OK) return r;
  WG_ON_DEVICE(device);
  const wb_kernel_entry* k = wb_kernel_at(li.kernel_id);
  CUtensorMap map_a, map_b, map_c, map_cw;
  std::memset(&map_c, 0, sizeof map_c);
  std::memset(&map_cw, 0, sizeof map_cw);
  if ((r = encode_2d(&map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, dA, M, K, li.a_box_rows, 64)) != WG_OK) return r;
  if ((r = encode_2d(&map_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, dBt, N, K, li.bt_box_rows, 64)) != WG_OK) return r;
  if (!li.direct && (r = encode_2d(&map_c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dC, M, N, li.c_box_rows, 32, CU_TENSOR_MAP_SWIZZLE_NONE)) != WG_OK) return r;
  if (!li.direct && (r = encode_2d(&map_cw, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dC, M, N, k->wide_rows, 32, CU_TENSOR_MAP_SWIZZLE_NONE)) != WG_OK) return r;
  KParams p;
  std::memset(&p, 0, sizeof p);
  p.M = M, p.N = N, p.K = K, p.ldc = N, p.kt = K / 64;
  p.ntiles = ((M + li.tile_m - 1) / li.tile_m) * ((N + li.tile_n - 1) / li.tile_n);
  p.cl_n = li.cl_n > 0 ? li.cl_n : 1, p.group = li.group > 0 ? li.group : 1, p.serp = li.serpentine;
  p.depth = li.depth, p.nbuf = li.nbuf, p.sched = li.sched, p.ask_ahead = li.ask_ahead, p.split = li.split;
  p.ksub = li.ksub, p.rounds = li.rounds;
  p.l2_hints = l2_hints_for(li, M, N, K);
  p.staging_bytes = li.staging_bytes;
  p.late_launch = v->late_launch;
  p.epi_ring = li.wide_rows != 0;
  if (li.sched == SCHED_STREAMK) {
    const int clusters = li.grid / li.cluster, units = (p.ntiles / li.cluster - li.sk_dp) * p.kt;
    p.sk_clusters = clusters, p.sk_q = units / clusters, p.sk_r = units % clusters, p.sk_dp = li.sk_dp;
  }
  p.C = static_cast<float*>(dC);
  p.status = scratch;      // 8 status words, then the flags
  p.flags = scratch + 8;
  p.timeout_ns = 2000ull * 1000ull * 1000ull;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  // the array keeps the last call's contents and the flags of one launch must all start equal:
  // clear the words this launch uses (and the status) on the stream, ahead of the kernel
  WG_CUDA(cudaMemsetAsync(scratch, 0, size_t(8 + (li.nflags > 0 ? li.nflags : 0)) * sizeof(uint32_t), stream));
  WG_CUDA(cudaFuncSetAttribute(k->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem));
  if ((r = check_coresident(k, li)) != WG_OK) return r;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  launch_config(li, stream, false, &cfg, attr);
  void* args[5] = {&map_a, &map_b, &map_c, &map_cw, &p};
  return int(cudaLaunchKernelExC(&cfg, k->fn, args));
}

extern "C" int wg_noalloc_status(int device, unsigned out[4]) {
  if (!out) return WG_E_ARG;
  uint32_t* scratch = nullptr;
  const int r = noalloc_setup(device, &scratch);
  if (r != WG_OK) return r;
  uint32_t st[4];
  WG_ON_DEVICE(device);
  WG_CUDA(cudaDeviceSynchronize());
  WG_CUDA(cudaMemcpy(st, scratch, sizeof st, cudaMemcpyDeviceToHost));
  for (int i = 0; i < 4; ++i) out[i] = st[i];
  return st[0] == 0 ? WG_OK : WG_E_DEVICE_WAIT;
}

// Bits 8-11 choose how many k-steps the ring hands over per barrier round (results stay exact).
// Bits 0-7 exist only in builds with -DWB_TIMING_EXPERIMENTS (bit 0: the producer loads nothing,
// bit 1: no MMAs are issued, bits 4-5: flip the L2 hints; results are then meaningless); the
// library as shipped refuses them.
extern "C" int wg_plan_debug_set_mode(void* plan, unsigned flags) {
  Plan* pl = static_cast<Plan*>(plan);
  if (!pl) return WG_E_ARG;
#ifdef WB_TIMING_EXPERIMENTS
  pl->p.debug = flags & 0xffu;
#else
  if (flags & 0xffu) return WG_E_ARG;
#endif
  // bits 8-11: k-steps a barrier round (1, 2 or 4) for the launches that follow; 0 = the library's choice
  const int ksub = int((flags >> 8) & 0xfu);
  if (ksub == 0) pl->p.ksub = pl->li.ksub, pl->p.rounds = pl->li.rounds;
  else if ((ksub == 1 || ((ksub == 2 || ksub == 4) && pl->k->reps == 1)) && pl->p.depth / ksub >= 2) pl->p.ksub = ksub, pl->p.rounds = pl->p.depth / ksub;
  else return WG_E_ARG;
  return WG_OK;
}
