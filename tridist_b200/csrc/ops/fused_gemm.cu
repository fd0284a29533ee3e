// Host side of the fused GEMM family: TMA descriptor encoding, plan objects
// (one pre-built parameter block per workspace parity) and launches.
#include "fused_gemm.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <array>
#include <mutex>
#include <stdexcept>
#include <vector>
#include <string>
#include <unordered_map>

#include "../gemm/fused_gemm.cuh"

namespace tdb {

static void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess)
    throw std::runtime_error(std::string("tridist_b200: ") + what + ": " + cudaGetErrorString(e));
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    check(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q),
          "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
    if (q != cudaDriverEntryPointSuccess || p == nullptr)
      throw std::runtime_error("tridist_b200: cuTensorMapEncodeTiled is not available");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Row-major [rows, cols] 16-bit matrix, box = 128 rows x 64 columns, 128-byte swizzle.
static CUtensorMap make_tmap(const void* base, int64_t rows, int64_t cols, int64_t row_stride_elems,
                             bool bf16, int box_rows = 128) {
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0)
    throw std::runtime_error("tridist_b200: TMA base address must be 16-byte aligned");
  if ((row_stride_elems * 2) % 16 != 0)
    throw std::runtime_error("tridist_b200: TMA row stride must be a multiple of 16 bytes");
  CUtensorMap m;
  const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(row_stride_elems) * 2};
  const cuuint32_t box[2] = {BK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = encode_fn()(&m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                           2, const_cast<void*>(base), gdim, gstride, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    throw std::runtime_error("tridist_b200: cuTensorMapEncodeTiled failed with code " +
                             std::to_string(static_cast<int>(r)));
  return m;
}

struct GemmPlan {
  GemmParams prm[2];
  int bn;
  bool bf16;
  int cta_m;
  int cta_mt;
  int grid_x;
  GemmParams* dev_params = nullptr;   // emulated multi-rank launches only
};

static int resident_ctas_of(const GemmPlan& plan);

static std::mutex g_mu;
static std::unordered_map<int64_t, GemmPlan*> g_plans;
static int64_t g_next_plan = 1;
static int64_t g_launches = 0;

int64_t launch_count() { return g_launches; }
void launch_count_add(int64_t n) { g_launches += n; }

static int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    check(cudaGetDevice(&dev), "cudaGetDevice");
    check(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev), "SM count");
  }
  return n;
}

template <int BN, bool kBf16, int kCtaM, bool kStaging, int kMT>
static void set_attr_once() {
  static bool done = false;
  if (!done) {
    check(cudaFuncSetAttribute(fused_gemm_kernel<BN, kBf16, kCtaM, kStaging, kMT>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                               TileShape<BN, kCtaM, kStaging, kMT>::kSmemBytes),
          "cudaFuncSetAttribute(smem)");
    done = true;
  }
}

// CTA pairs (one 2-CTA tcgen05 MMA per 256-wide output tile) where the schedule allows.
static int choose_cta_m(const GemmPlanDesc& d) {
  const int mt = (d.M + BM - 1) / BM;
  bool pair = d.allow_pair && d.bn == 256 && mt >= 2 && d.sched != SCHED_LIST;
  if (d.sched == SCHED_SEGMENT && ((mt / d.R) % 2 != 0)) pair = false;
  return pair ? 2 : 1;
}

// 128-row blocks per CTA: 2 (a 512 x 256 tile per CTA pair) where there are enough rows and the
// schedule's row segments are whole numbers of such tiles.
static int choose_cta_mt(const GemmPlanDesc& d, int cta_m) {
  const int mt = (d.M + BM - 1) / BM;
  if (cta_m != 2 || !d.allow_wide || mt < 4) return 1;
  if (d.sched == SCHED_SEGMENT && ((mt / d.R) % 4 != 0)) return 1;
  // reduce-scatter tiles whose rows belong to several owners keep the 128-row granularity
  if (d.op == OP_RS && d.R > 1 && d.sched != SCHED_SEGMENT) return 1;
  return 2;
}

constexpr int kMinKBlocksPerSlice = 8;    // a K range shorter than this is not worth a partial

// Everything the tile schedule depends on (shared by plan creation and the host-side dump).
static void fill_schedule_fields(const GemmPlanDesc& d, int cta_m, int cta_mt, GemmParams& p) {
  const int bn_out = (d.epi == EPI_SWIGLU) ? d.bn / 2 : d.bn;
  p.M = d.M; p.N = d.N; p.K = d.K;
  p.m_tiles = (d.M + BM - 1) / BM;
  p.n_tiles = (d.N + bn_out - 1) / bn_out;
  p.k_blocks = (d.K + BK - 1) / BK;
  p.rank = d.rank; p.R = d.R;
  p.op = d.op; p.epi = d.epi; p.sched = d.sched;
  p.m_per_rank = d.m_per_rank > 0 ? d.m_per_rank : d.M;
  p.cta_m = cta_m;
  p.cta_mt = cta_mt;
  p.sub_tiles = cta_m * cta_mt;
  p.unit_m = (p.m_tiles + p.sub_tiles - 1) / p.sub_tiles;
  p.seg_m_tiles = (d.sched == SCHED_SEGMENT) ? (p.m_tiles / d.R) / p.sub_tiles : p.unit_m;
  // row units walked together: their A rows (unit rows x K) should stay in L2 while the B column
  // blocks stream past, and a wave of workers should still span several column blocks
  {
    const int64_t unit_bytes = static_cast<int64_t>(p.sub_tiles) * BM * d.K * 2;
    int g = d.raster_g > 0 ? d.raster_g : static_cast<int>((48ll << 20) / (unit_bytes > 0 ? unit_bytes : 1));
    if (g < 1) g = 1;
    if (g > 16) g = 16;
    p.raster_g = g;
  }
  if (d.sched == SCHED_SEGMENT && (p.m_tiles % d.R != 0 || p.m_per_rank % BM != 0))
    throw std::runtime_error("tridist_b200: segment order needs rows per rank % 128 == 0");
  for (int i = 0; i < kMaxRanks; ++i) p.seg_order[i] = (i < d.R) ? d.seg_order[i] : 0;
  p.strided_interleave = d.strided_interleave;
  p.seg_interleave = (d.sched == SCHED_SEGMENT) ? d.seg_interleave : 0;
  p.seg_bands = (d.sched == SCHED_SEGMENT && d.seg_bands > 1) ? d.seg_bands : 1;
  // seg_bands < 0: as many bands as a segment has row units (one unit per band)
  if (d.sched == SCHED_SEGMENT && d.seg_bands < 0 && p.seg_m_tiles > 1) p.seg_bands = p.seg_m_tiles;
  p.seg_own_first = (d.seg_own_first && p.seg_bands > 1) ? 1 : 0;
  p.list_len = d.list_len;
  p.swiglu_up_row0 = d.swiglu_up_row0;
  p.chunk_rows = d.chunk_rows > 0 ? d.chunk_rows : p.m_per_rank;
  p.n_chunks = d.n_chunks > 0 ? d.n_chunks : 1;
  p.push_parts = d.push_parts > 0 ? d.push_parts : 1;
  p.skip_comm = d.skip_comm;
  p.push_ctas = d.push_ctas;
  p.push_skip_rounds = d.push_skip_rounds;
  const int own_tickets = p.unit_m * p.sub_tiles * p.n_tiles;
  if (d.ticket_stride > 0 && d.ticket_stride < own_tickets)
    throw std::runtime_error("tridist_b200: ticket stride " + std::to_string(d.ticket_stride) +
                             " is smaller than this call's " + std::to_string(own_tickets) + " tile tickets");
  if (d.ag_flag_stride > 0 && d.ag_flag_stride < p.n_chunks)
    throw std::runtime_error("tridist_b200: chunk-ticket stride is smaller than this call's chunk count");
  p.ticket_stride = d.ticket_stride > 0 ? d.ticket_stride : own_tickets;
  p.ag_flag_stride = d.ag_flag_stride > 0 ? d.ag_flag_stride : p.n_chunks;
}

// Persistent grid: one CTA (or CTA pair) per scheduling position, at most one per SM; and the
// split of the last, partial round along K (fills p.sk_tiles / p.sk_slices).
static int grid_for(const GemmPlanDesc& d, GemmParams& p, int max_ctas, int sms) {
  const int positions = sched_positions(p);
  int g = max_ctas > 0 ? max_ctas : sms;
  if (g > sms) g = sms;
  g /= p.cta_m;                             // workers that can run at once
  if (g < 1) g = 1;
  p.sk_tiles = 0;
  p.sk_slices = 1;
  const bool may_split = d.allow_splitk && d.sched != SCHED_LIST && d.probe == 0 && positions > 0;
  int slices_cap = p.k_blocks / kMinKBlocksPerSlice;
  if (slices_cap > kMaxSlices) slices_cap = kMaxSlices;
  int workers;
  if (positions < g) {
    // fewer tiles than workers (skinny M): every tile is cut
    int s = may_split ? g / positions : 1;
    if (s > slices_cap) s = slices_cap;
    if (s >= 2) {
      p.sk_tiles = positions;
      p.sk_slices = s;
      workers = positions * s;
    } else {
      workers = positions < 1 ? 1 : positions;
    }
  } else {
    workers = g;
    int pushers = 0, skip = 0;
    if (d.op == OP_AG && d.R > 1 && !d.skip_comm && d.push_ctas > 0 && d.push_ctas < workers * p.cta_m) {
      pushers = (d.push_ctas + p.cta_m - 1) / p.cta_m;
      skip = d.push_skip_rounds;
    }
    const int r = remainder_positions(positions, workers, pushers, skip);
    int s = (may_split && r > 0) ? workers / r : 1;
    if (s > slices_cap) s = slices_cap;
    if (s >= 2) {
      p.sk_tiles = r;
      p.sk_slices = s;
    }
  }
  return workers * p.cta_m;
}

// Scratch for the split-K partials: one slot per CTA of a launch (two fp32 accumulators of
// 128 x 256) and one epoch word per slot; allocated once per device, on first use, never freed.
constexpr int kSkSlots = 160;
constexpr int64_t kSkSlotWords = 2ll * BM * 256;
struct SkScratch {
  float* ws = nullptr;
  uint32_t* flags = nullptr;
};
static SkScratch& sk_scratch() {
  static SkScratch per_dev[64];
  int dev = 0;
  check(cudaGetDevice(&dev), "cudaGetDevice");
  SkScratch& s = per_dev[dev & 63];
  if (s.ws == nullptr) {
    check(cudaMalloc(&s.ws, kSkSlots * kSkSlotWords * sizeof(float)), "cudaMalloc(split-K scratch)");
    check(cudaMalloc(&s.flags, kSkSlots * sizeof(uint32_t)), "cudaMalloc(split-K flags)");
    check(cudaMemset(s.flags, 0, kSkSlots * sizeof(uint32_t)), "cudaMemset(split-K flags)");
  }
  return s;
}
static uint32_t g_sk_epoch = 0;

std::vector<std::vector<std::array<int, 5>>> schedule_dump(const GemmPlanDesc& d, int sms) {
  if (d.sched == SCHED_LIST) throw std::runtime_error("tridist_b200: a tile list is its own schedule");
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  const int cta_m = choose_cta_m(d);
  fill_schedule_fields(d, cta_m, choose_cta_mt(d, cta_m), p);
  const int grid_x = grid_for(d, p, d.max_ctas, sms);
  const WorkerSchedule ws = make_worker_schedule(p, grid_x, cta_m);
  std::vector<std::vector<std::array<int, 5>>> out(grid_x);
  for (int cta = 0; cta < grid_x; ++cta) {
    const int sub = cta % cta_m, worker = cta / cta_m;
    WorkIter wit;
    WorkItem wi;
    while (wit.next(ws, worker, p.k_blocks, wi)) {
      const TileCoord t = tile_at(p, p.seg_order, wi.pos, sub, p.seg_bands);
      if (!t.valid) continue;
      // a tile cut along K appears once, with the worker that finishes it (slice 0)
      if (wi.slice > 0) continue;
      for (int h = 0; h < p.cta_mt; ++h)
        out[cta].push_back({t.m_tile + h, t.n_tile, tile_linear(p, t, h), t.owner_key, wi.pos});
    }
  }
  return out;
}

// The K ranges of the tiles that are cut along K: {scheduling position, first CTA of the worker,
// slice, slices, first k-block, end k-block} for every worker that takes part.
std::vector<std::array<int, 6>> splitk_dump(const GemmPlanDesc& d, int sms) {
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  const int cta_m = choose_cta_m(d);
  fill_schedule_fields(d, cta_m, choose_cta_mt(d, cta_m), p);
  const int grid_x = grid_for(d, p, d.max_ctas, sms);
  const WorkerSchedule ws = make_worker_schedule(p, grid_x, cta_m);
  std::vector<std::array<int, 6>> out;
  for (int worker = 0; worker < grid_x / cta_m; ++worker) {
    WorkIter wit;
    WorkItem wi;
    while (wit.next(ws, worker, p.k_blocks, wi))
      if (wi.slices > 1) out.push_back({wi.pos, worker * cta_m, wi.slice, wi.slices, wi.kb0, wi.kb1});
  }
  return out;
}

std::vector<std::string> plan_check(const GemmPlanDesc& d, const PlanExtents& e, int sms) {
  std::vector<std::string> bad;
  auto need = [&](const char* what, int64_t want, int64_t have, const char* unit) {
    if (have > 0 && want > have)
      bad.push_back(std::string(what) + " needs " + std::to_string(want) + " " + unit + ", has " +
                    std::to_string(have));
  };
  if (d.sched == SCHED_LIST) return bad;      // a tile list is checked against the grid by its maker
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  const int cta_m = choose_cta_m(d);
  try {
    fill_schedule_fields(d, cta_m, choose_cta_mt(d, cta_m), p);
  } catch (const std::exception& ex) {
    bad.push_back(ex.what());
    return bad;
  }
  const bool multi = d.R > 1;
  // ---- tiles and tickets: every tile once, ticket indices unique and inside the ticket planes ----
  const int64_t tickets = (d.sched == SCHED_STRIDED)
      ? static_cast<int64_t>(p.unit_m) * p.sub_tiles * p.n_tiles
      : static_cast<int64_t>(p.m_tiles) * p.n_tiles;
  const auto sched = schedule_dump(d, sms);
  std::vector<char> seen(static_cast<size_t>(p.unit_m) * p.sub_tiles * p.n_tiles, 0);
  std::vector<char> ticket_used(static_cast<size_t>(tickets > 0 ? tickets : 1), 0);
  int64_t real_tiles = 0;
  for (const auto& cta : sched) {
    for (const auto& t : cta) {
      const int mt = t[0], nt = t[1], lin = t[2];
      if (mt < 0 || mt >= p.unit_m * p.sub_tiles || nt < 0 || nt >= p.n_tiles) {
        bad.push_back("tile (" + std::to_string(mt) + ", " + std::to_string(nt) + ") outside the tile grid");
        continue;
      }
      // the second CTA of the last pair can stand past the last row block (odd number of row
      // blocks): such a tile has no rows, the kernel touches no ticket for it
      const bool has_rows = mt < p.m_tiles;
      if ((has_rows || d.sched == SCHED_STRIDED) && (lin < 0 || lin >= tickets))
        bad.push_back("ticket index " + std::to_string(lin) + " outside [0, " + std::to_string(tickets) + ")");
      if ((has_rows || d.sched == SCHED_STRIDED) && lin >= 0 && lin < tickets) {
        if (ticket_used[lin]) bad.push_back("ticket index " + std::to_string(lin) + " used by two tiles");
        ticket_used[lin] = 1;
      }
      char& s = seen[static_cast<size_t>(mt) * p.n_tiles + nt];
      if (s) bad.push_back("tile (" + std::to_string(mt) + ", " + std::to_string(nt) + ") scheduled twice");
      s = 1;
      if (mt < p.m_tiles) ++real_tiles;
    }
  }
  if (real_tiles != static_cast<int64_t>(p.m_tiles) * p.n_tiles)
    bad.push_back("schedule covers " + std::to_string(real_tiles) + " of " +
                  std::to_string(static_cast<int64_t>(p.m_tiles) * p.n_tiles) + " tiles");
  // ---- buffers ------------------------------------------------------------------------------
  const int64_t out_rows = (multi && d.op == OP_RS) ? p.m_per_rank : d.M;
  const int64_t out_cols = d.N;
  need("output c", ((out_rows - 1) * d.ldc + out_cols) * 2, e.c_bytes, "bytes");
  if (multi && d.op == OP_AG) {
    need("all-gather workspace", static_cast<int64_t>(d.M) * d.K * 2, e.ws_bytes, "bytes");
    need("all-gather ticket plane", static_cast<int64_t>(d.R - 1) * p.ag_flag_stride + p.n_chunks,
         e.ag_flag_words, "words");
    if (static_cast<int64_t>(p.chunk_rows) * p.n_chunks != p.m_per_rank)
      bad.push_back("chunk_rows * n_chunks differs from the rows per rank");
    if (static_cast<int64_t>(p.m_per_rank) * d.R != d.M)
      bad.push_back("rows per rank * ranks differs from M");
  }
  if (multi && (d.op == OP_RS || d.op == OP_AR1 || d.op == OP_AR2)) {
    const int64_t plane = ((d.op == OP_RS && !d.nvls) ? static_cast<int64_t>(p.m_per_rank) : d.M) * d.N;
    need(d.nvls ? "local partial plane" : "partial slots",
         (static_cast<int64_t>(d.R - 1) * d.slot_stride * (d.nvls ? 0 : 1) + plane) * 2, e.slot_bytes, "bytes");
    if (!d.nvls && d.slot_stride < plane)
      bad.push_back("slot stride " + std::to_string(d.slot_stride) + " is smaller than one slot (" +
                    std::to_string(plane) + " elements)");
    need("tile ticket plane", static_cast<int64_t>(d.R - 1) * p.ticket_stride + tickets, e.tile_flag_words,
         "words");
    if (d.op == OP_RS && static_cast<int64_t>(p.m_per_rank) * d.R != d.M)
      bad.push_back("rows per rank * ranks differs from M");
  }
  if (multi && d.op == OP_AR2) {
    need("result plane", static_cast<int64_t>(d.M) * d.N * 2, e.res_bytes, "bytes");
    need("result ticket plane", static_cast<int64_t>(d.R - 1) * p.ticket_stride + tickets, e.res_flag_words,
         "words");
  }
  return bad;
}

int64_t gemm_plan_create(const GemmPlanDesc& d) {
  if (d.R < 1 || d.R > kMaxRanks) throw std::runtime_error("tridist_b200: 1 <= R <= 8 required");
  if (d.bn != 128 && d.bn != 256) throw std::runtime_error("tridist_b200: BN must be 128 or 256");
  if (d.epi == EPI_SWIGLU && d.bn != 256)
    throw std::runtime_error("tridist_b200: the SwiGLU epilogue needs BN = 256");
  if (d.R > 1 && (d.op == OP_RS || d.op == OP_AR1 || d.op == OP_AR2) && d.N % 128 != 0)
    throw std::runtime_error("tridist_b200: GEMM+RS / GEMM+AR need N % 128 == 0");
  if (d.op == OP_AR2 && d.R > 1 && d.ldc % 8 != 0)
    throw std::runtime_error("tridist_b200: GEMM+AR needs a 16-byte aligned row stride of c");
  if (d.nvls && d.op == OP_AR2 && d.R > 1) {
    if (d.slot_stride != 0) throw std::runtime_error("tridist_b200: switch-reduced all-reduce keeps partials local (slot_stride = 0)");
    for (int par = 0; par < 2; ++par)
      if (d.mc_part[par] == 0 || d.mc_res[par] == 0 || d.mc_part[par] % 16 != 0 || d.mc_res[par] % 16 != 0)
        throw std::runtime_error("tridist_b200: switch-reduced all-reduce needs 16-byte aligned multicast addresses");
  }
  if (d.nvls && d.op == OP_RS && d.R > 1) {
    if (d.slot_stride != 0 || d.sched != SCHED_SEGMENT || !d.seg_interleave)
      throw std::runtime_error("tridist_b200: switch-reduced reduce-scatter keeps partials local (slot_stride = 0) "
                               "and walks the owners' segments in lockstep");
    if (d.ldc % 8 != 0 || d.c % 16 != 0)
      throw std::runtime_error("tridist_b200: switch-reduced reduce-scatter needs a 16-byte aligned c");
    for (int par = 0; par < 2; ++par)
      if (d.mc_part[par] == 0 || d.mc_part[par] % 16 != 0)
        throw std::runtime_error("tridist_b200: switch-reduced reduce-scatter needs a 16-byte aligned multicast address");
  }
  if (d.K % 8 != 0) throw std::runtime_error("tridist_b200: K must be a multiple of 8");
  if (d.N % 8 != 0) throw std::runtime_error("tridist_b200: N must be a multiple of 8");
  auto* plan = new GemmPlan();
  plan->bn = d.bn;
  plan->bf16 = d.bf16;
  plan->cta_m = choose_cta_m(d);
  plan->cta_mt = choose_cta_mt(d, plan->cta_m);
  for (int par = 0; par < 2; ++par) {
    GemmParams& p = plan->prm[par];
    std::memset(&p, 0, sizeof(p));
    fill_schedule_fields(d, plan->cta_m, plan->cta_mt, p);
    p.order_table = reinterpret_cast<const int32_t*>(d.order_table);
    p.table_has_header = (d.order_table != 0 && d.order_table_header) ? 1 : 0;
    p.tile_list = reinterpret_cast<const int32_t*>(d.tile_list);
    p.is_bf16 = d.bf16 ? 1 : 0;
    p.c = reinterpret_cast<void*>(d.c);
    p.ldc = d.ldc;
    // tiles that stay on this GPU leave through staged TMA stores when c can carry a tensor map
    p.c_tma = 0;
    if (d.c != 0 && d.c % 16 == 0 && (d.ldc * 2) % 16 == 0 && (d.R == 1 || d.op == OP_PLAIN || d.op == OP_AG)) {
      p.tma_c32 = make_tmap(reinterpret_cast<void*>(d.c), d.M, d.N, d.ldc, d.bf16, 32);
      p.c_tma = 1;
    }
    p.tma_a = make_tmap(reinterpret_cast<void*>(d.a), d.a_rows, d.K, d.lda, d.bf16);
    p.tma_b = make_tmap(reinterpret_cast<void*>(d.b), d.b_rows, d.K, d.ldb, d.bf16);
    p.tma_a_ws = p.tma_a;
    p.a_local = reinterpret_cast<const void*>(d.a);
    p.ag_counters = reinterpret_cast<uint32_t*>(d.ag_counters);
    p.ag_pull = (d.ag_pull && d.op == OP_AG && d.R > 1) ? 1 : 0;
    if (p.ag_pull)
      for (int r = 0; r < d.R; ++r)
        if (d.peer_ag_arrive[r] == 0) throw std::runtime_error("tridist_b200: pull all-gather needs the arrive ticket plane");
    p.arrival_ns = reinterpret_cast<uint64_t*>(d.arrival_ns);
    p.slot_stride = d.slot_stride;
    p.res_is_c = d.res_is_c;
    p.nvls = (d.nvls && (d.op == OP_AR2 || d.op == OP_RS) && d.R > 1) ? 1 : 0;
    p.ag_mc = (d.nvls && d.op == OP_AG && d.R > 1 && !p.ag_pull) ? 1 : 0;
    p.l2_ahead = d.l2_ahead < 0 ? 0 : (d.l2_ahead > 32 ? 32 : d.l2_ahead);
    if (p.ag_mc && (d.mc_part[par] == 0 || d.mc_part[par] % 16 != 0 || d.K % 8 != 0))
      throw std::runtime_error("tridist_b200: multicast all-gather needs a 16-byte aligned multicast workspace address");
    p.reduce_ctas = d.reduce_ctas;
    p.reduce_tail = d.reduce_tail;
    p.mc_part = reinterpret_cast<void*>(d.mc_part[par]);
    p.mc_res = reinterpret_cast<void*>(d.mc_res[par]);
    for (int r = 0; r < d.R; ++r) {
      p.peer_ws[r] = reinterpret_cast<void*>(d.peer_ws[par][r]);
      p.peer_ag_flags[r] = reinterpret_cast<uint32_t*>(d.peer_ag_flags[r]);
      p.peer_ag_arrive[r] = reinterpret_cast<uint32_t*>(d.peer_ag_arrive[r]);
      p.peer_slots[r] = reinterpret_cast<void*>(d.peer_slots[par][r]);
      p.peer_tile_flags[r] = reinterpret_cast<uint32_t*>(d.peer_tile_flags[r]);
      p.peer_res[r] = reinterpret_cast<void*>(d.peer_res[par][r]);
      p.peer_res_flags[r] = reinterpret_cast<uint32_t*>(d.peer_res_flags[r]);
    }
    if (d.op == OP_AG && d.R > 1) {
      if (((static_cast<int64_t>(p.chunk_rows) * d.K * 2) / p.push_parts) % 16 != 0)
        throw std::runtime_error("tridist_b200: AG push part size must be a multiple of 16 bytes");
      p.tma_a_ws = make_tmap(p.peer_ws[d.rank], d.M, d.K, d.K, d.bf16);
    }
    if (d.R > 1 && (d.op == OP_RS || d.op == OP_AR1 || d.op == OP_AR2)) {
      // store maps over this rank's slot inside every rank's slot buffer
      const int64_t slot_rows = (d.op == OP_RS && !p.nvls) ? p.m_per_rank : d.M;
      for (int r = 0; r < d.R; ++r) {
        uint8_t* base = reinterpret_cast<uint8_t*>(p.peer_slots[r]) +
                        static_cast<int64_t>(d.rank) * d.slot_stride * 2;
        p.tma_slot[r] = make_tmap(base, slot_rows, d.N, d.N, d.bf16);
      }
    }
    p.prof = reinterpret_cast<uint64_t*>(d.prof);
    p.env.status = reinterpret_cast<StatusBlock*>(d.status_dev);
    p.env.abort_word = reinterpret_cast<uint32_t*>(d.abort_word);
    p.env.n_peers = 0;
    for (int r = 0; r < kMaxRanks; ++r) {
      p.env.peer_abort[r] = reinterpret_cast<uint32_t*>(d.peer_abort[r]);
      if (d.peer_abort[r] != 0) p.env.n_peers = static_cast<uint32_t>(r + 1);
    }
    p.env.timeout_ns = d.timeout_ns;
    p.env.poll_ns = d.poll_ns;
    p.probe = (d.op == OP_PLAIN && d.R == 1) ? d.probe : 0;
    p.env.rank = static_cast<uint32_t>(d.rank);
  }
  plan->grid_x = grid_for(d, plan->prm[0], d.max_ctas, num_sms());
  if (d.check_residency) {
    const int fit = resident_ctas_of(*plan);
    if (plan->grid_x > fit) {
      const int gx = plan->grid_x;
      delete plan;
      throw std::runtime_error("tridist_b200: the kernel's " + std::to_string(gx) + " CTAs wait on one another but only " +
                               std::to_string(fit) + " can be resident at once on this device (is another "
                               "kernel holding SMs or shared memory?)");
    }
  }
  plan->prm[1].sk_tiles = plan->prm[0].sk_tiles;
  plan->prm[1].sk_slices = plan->prm[0].sk_slices;
  if (plan->prm[0].sk_tiles > 0) {
    if (plan->grid_x > kSkSlots) throw std::runtime_error("tridist_b200: split-K scratch has too few slots");
    const SkScratch& sc = sk_scratch();
    for (int par = 0; par < 2; ++par) {
      plan->prm[par].sk_ws = sc.ws;
      plan->prm[par].sk_flags = sc.flags;
      plan->prm[par].sk_slot_words = plan->cta_mt * BM * plan->bn;
    }
  }
  std::lock_guard<std::mutex> lk(g_mu);
  const int64_t id = g_next_plan++;
  g_plans[id] = plan;
  return id;
}

void gemm_plan_destroy(int64_t id) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_plans.find(id);
  if (it == g_plans.end()) return;
  if (it->second->dev_params) cudaFree(it->second->dev_params);
  delete it->second;
  g_plans.erase(it);
}

static GemmPlan* find_plan(int64_t id) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_plans.find(id);
  if (it == g_plans.end()) throw std::runtime_error("tridist_b200: unknown GEMM plan");
  return it->second;
}

// CTAs of one variant that can be resident on the device at once (whole clusters for CTA pairs).
// The kernels wait on one another across CTAs and across ranks, so a grid that does not fit in
// one wave could wait for a CTA that is not running.
template <int BN, bool kBf16, int kCtaM, bool kStaging, int kMT>
static int resident_ctas() {
  static int cached = -1;
  if (cached >= 0) return cached;
  set_attr_once<BN, kBf16, kCtaM, kStaging, kMT>();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(num_sms() / kCtaM * kCtaM, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = TileShape<BN, kCtaM, kStaging, kMT>::kSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCtaM;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  check(cudaOccupancyMaxActiveClusters(&clusters, fused_gemm_kernel<BN, kBf16, kCtaM, kStaging, kMT>, &cfg),
        "cudaOccupancyMaxActiveClusters");
  cached = clusters * kCtaM;
  return cached;
}

static bool plan_uses_staging(const GemmParams& p) {
  // operators that ship data to other ranks (epilogue tiles, all-gather push) need the staging area
  return p.R > 1 && (p.op == OP_RS || p.op == OP_AR1 || p.op == OP_AR2 || p.op == OP_AG);
}

static int resident_ctas_of(const GemmPlan& plan) {
  const bool st = plan_uses_staging(plan.prm[0]);
#define TDB_RES(BN_, PAIR_, MT_)                                                            \
  (plan.bf16 ? (st ? resident_ctas<BN_, true, PAIR_, true, MT_>() : resident_ctas<BN_, true, PAIR_, (MT_ == 2), MT_>()) \
             : (st ? resident_ctas<BN_, false, PAIR_, true, MT_>() : resident_ctas<BN_, false, PAIR_, (MT_ == 2), MT_>()))
  if (plan.bn == 256) {
    if (plan.cta_m == 2 && plan.cta_mt == 2) return TDB_RES(256, 2, 2);
    if (plan.cta_m == 2) return TDB_RES(256, 2, 1);
    return TDB_RES(256, 1, 1);
  }
  return TDB_RES(128, 1, 1);
#undef TDB_RES
}

template <int BN, bool kBf16, int kCtaM, bool kStaging, int kMT>
static void launch_one(const GemmParams& p, int grid_x, cudaStream_t stream) {
  set_attr_once<BN, kBf16, kCtaM, kStaging, kMT>();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid_x, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = TileShape<BN, kCtaM, kStaging, kMT>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCtaM;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const GemmParams* none = nullptr;
  check(cudaLaunchKernelEx(&cfg, fused_gemm_kernel<BN, kBf16, kCtaM, kStaging, kMT>, p, none),
        "fused_gemm_kernel launch");
}

void gemm_plan_launch(int64_t id, uint32_t round, int parity, int64_t order_table, int flags,
                      void* stream_) {
  GemmPlan* plan = find_plan(id);
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  GemmParams& p = plan->prm[parity & 1];
  p.round = round;
  p.order_table = reinterpret_cast<const int32_t*>(order_table);
  p.table_has_header = (order_table != 0 && ((flags >> 3) & 1)) ? 1 : 0;
  p.skip_comm = flags & 1;
  p.comm_only = (flags >> 1) & 1;
  p.publish_only = (flags >> 2) & 1;
  p.sk_epoch = ++g_sk_epoch;
  const bool staging = plan_uses_staging(p);
#define TDB_LAUNCH(BN_, PAIR_)                                                              \
  do {                                                                                      \
    if (plan->bf16) {                                                                       \
      if (staging) launch_one<BN_, true, PAIR_, true, 1>(p, plan->grid_x, stream);          \
      else launch_one<BN_, true, PAIR_, false, 1>(p, plan->grid_x, stream);                 \
    } else {                                                                                \
      if (staging) launch_one<BN_, false, PAIR_, true, 1>(p, plan->grid_x, stream);         \
      else launch_one<BN_, false, PAIR_, false, 1>(p, plan->grid_x, stream);                \
    }                                                                                       \
  } while (0)
  if (plan->bn == 256) {
    if (plan->cta_m == 2 && plan->cta_mt == 2) {
      // 256 rows per CTA: the ring has four stages and the staging area is always there
      if (plan->bf16) launch_one<256, true, 2, true, 2>(p, plan->grid_x, stream);
      else launch_one<256, false, 2, true, 2>(p, plan->grid_x, stream);
    } else if (plan->cta_m == 2) {
      TDB_LAUNCH(256, 2);
    } else {
      TDB_LAUNCH(256, 1);
    }
  } else {
    TDB_LAUNCH(128, 1);
  }
#undef TDB_LAUNCH
  ++g_launches;
}

template <int BN, bool kBf16, int kCtaM, int kMT>
static void launch_emulated(const GemmParams* dev, int grid_x, int vranks, cudaStream_t stream) {
  set_attr_once<BN, kBf16, kCtaM, true, kMT>();
  GemmParams dummy;
  std::memset(&dummy, 0, sizeof(dummy));
  // Cooperative launch: the runtime refuses the launch unless every CTA (every CTA pair) of
  // every emulated rank can be resident at once, which the cross-rank waits need.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid_x, vranks, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = TileShape<BN, kCtaM, true, kMT>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = kCtaM;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  check(cudaLaunchKernelEx(&cfg, fused_gemm_kernel<BN, kBf16, kCtaM, true, kMT>, dummy, dev),
        "fused_gemm_kernel cooperative launch");
}

// `skip_comm`: bit 0 = every rank skips its communication (GEMM-only decomposition); bit 8 + r =
// virtual rank r alone neither pushes nor waits (the others then wait for it in vain: the bounded
// wait runs out, which is how the give-up path is exercised on one GPU).
void gemm_plans_launch_emulated(const std::vector<int64_t>& ids, uint32_t round, int parity,
                                int skip_comm, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const int vr = static_cast<int>(ids.size());
  if (vr < 1 || vr > kMaxRanks) throw std::runtime_error("tridist_b200: bad emulated rank count");
  GemmPlan* first = find_plan(ids[0]);
  std::vector<GemmParams> host(vr);
  int grid_x = (num_sms() / vr) / first->cta_m * first->cta_m;
  for (int i = 0; i < vr; ++i) {
    GemmPlan* pl = find_plan(ids[i]);
    if (pl->bn != first->bn || pl->bf16 != first->bf16 || pl->cta_m != first->cta_m || pl->cta_mt != first->cta_mt)
      throw std::runtime_error("tridist_b200: emulated ranks must share the kernel variant");
    host[i] = pl->prm[parity & 1];
    host[i].round = round;
    host[i].skip_comm = (skip_comm & 1) | ((skip_comm >> (8 + i)) & 1);
    host[i].sk_epoch = g_sk_epoch + 1;
    if (pl->grid_x < grid_x) grid_x = pl->grid_x;
  }
  // the K split was laid out for each plan's own grid: a launch on a smaller grid deals whole tiles
  for (int i = 0; i < vr; ++i) {
    if (find_plan(ids[i])->grid_x != grid_x) {
      host[i].sk_tiles = 0;
      host[i].sk_slices = 1;
    }
  }
  if (!first->dev_params)
    check(cudaMalloc(&first->dev_params, sizeof(GemmParams) * kMaxRanks), "cudaMalloc(params)");
  check(cudaMemcpyAsync(first->dev_params, host.data(), sizeof(GemmParams) * vr,
                        cudaMemcpyHostToDevice, stream),
        "cudaMemcpyAsync(params)");
  check(cudaStreamSynchronize(stream), "cudaStreamSynchronize(params)");
#define TDB_EMU(BN_, CTAM_, MT_)                                                              \
  do {                                                                                        \
    if (first->bf16) launch_emulated<BN_, true, CTAM_, MT_>(first->dev_params, grid_x, vr, stream);  \
    else launch_emulated<BN_, false, CTAM_, MT_>(first->dev_params, grid_x, vr, stream);      \
  } while (0)
  if (first->bn == 256) {
    if (first->cta_m == 2 && first->cta_mt == 2) TDB_EMU(256, 2, 2);
    else if (first->cta_m == 2) TDB_EMU(256, 2, 1);
    else TDB_EMU(256, 1, 1);
  } else {
    TDB_EMU(128, 1, 1);
  }
#undef TDB_EMU
  ++g_sk_epoch;
  ++g_launches;
}

}  // namespace tdb
