// One persistent sm_100a kernel serves the plain GEMM and the three fused
// communication+GEMM operators:
//
//   OP_PLAIN   C = A @ B^T
//   OP_AG      C = allgather_M(A) @ B^T     comm warps push this rank's A shard into every
//                                           peer's workspace and raise per-(source, chunk)
//                                           tickets; the TMA warp gates each remote row
//                                           block on its ticket before loading it
//   OP_RS      out_r = rows r of sum_s A_s @ B_s^T
//                                           the epilogue stores partial tiles straight into
//                                           the owner rank's per-source slot; tiles of the
//                                           rank's own rows are reduced in the epilogue
//                                           (fp32) from the slots the peers filled; or, through
//                                           the switch: partial tiles stay in the producer's own
//                                           multicast-bound plane and the owner's communication
//                                           warps read their sum with multimem.ld_reduce
//   OP_AR1     one-shot all-reduce: every partial tile goes to all peers, each rank reduces
//   OP_AR2     two-shot all-reduce: every partial tile goes to the tile's owner; the owner's
//              communication warps reduce it and broadcast the result to all ranks
//
// Roles inside one CTA (320 threads, one CTA per SM):
//   warp 0      TMA producer (one lane): smem ring of kStages {A (kMT x 128) x 64, B x 64} tiles
//   warp 1      tcgen05.mma issuer (one lane), owns the TMEM allocation (2 accumulators)
//   warps 2-5   epilogue: tcgen05.ld -> convert -> staged TMA stores / peer stores (+ in-epilogue reduce)
//   warps 6-9   communication warps (AG push; AR2 reduce + broadcast + result collection)
//
// Tile shapes (template parameters kCtaM = CTAs per MMA, kMT = 128-row blocks per CTA):
//   kCtaM 1, kMT 1   128 x BN per CTA; the two TMEM accumulators double-buffer whole tiles
//   kCtaM 2, kMT 1   256 x 256 per CTA pair (cta_group::2), same double buffering
//   kCtaM 2, kMT 2   512 x 256 per CTA pair: every CTA holds 256 rows of A and its half of B per
//                    stage and issues two MMAs per K step, one per 128-row half, into the two
//                    accumulators. Three quarters of the operand bytes per FLOP of the 256 x 256
//                    pair tile (and of its shared-memory write traffic); the accumulators are no
//                    longer spare, so the epilogue drains half 0 first and the next tile's half-0
//                    MMAs start under the drain of half 1.
//
// Whole tiles are dealt round-robin to the workers (a worker = a CTA or a CTA pair). The tiles of
// the last, partial round are cut along K into `sk_slices` ranges, one per otherwise idle
// worker; slice 0 finishes the tile after adding the other slices' fp32 partials, which they
// park in a per-CTA scratch slot (split-K for the remainder wave and for skinny M).
//
// Reference behaviour covered (file paths inside the reference project):
//   triton_dist/kernels/dcu/all_gather_gemm.py:98-230   consumer GEMM gated on flags
//   triton_dist/kernels/dcu/all_gather_gemm.py:265-314  all-gather push + signalling
//   triton_dist/kernels/dcu/gemm_reduce_scatter.py:39-135 GEMM, scatter, reduce
//   triton_dist/kernels/dcu/gemm_allreduce.py:73-181    producer GEMM + consumer reduce
//   triton_dist/kernels/dcu/ag_tr_pred.py:344-361       table-driven tile order
//   bench/tune_gemm2.py:69-117                          split-K with fp32 accumulation
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../common/ptx.cuh"
#include "../common/sync.cuh"

namespace tdb {

constexpr int kMaxRanks = 8;
constexpr int BM = 128;
constexpr int BK = 64;            // 64 x 2 B = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 320;
constexpr int kEpiWarp0 = 2;
constexpr int kCommWarp0 = 6;
constexpr int kCommThreads = 128;
constexpr int kEpiThreads = 128;
constexpr int kMaxSlices = 8;     // K ranges a remainder tile can be cut into
constexpr int kPushSlots = 12;    // 16 KB pieces in flight per pushing CTA (all-gather)

enum GemmOp : int32_t { OP_PLAIN = 0, OP_AG = 1, OP_RS = 2, OP_AR1 = 3, OP_AR2 = 4 };
enum EpiMode : int32_t { EPI_STORE = 0, EPI_SWIGLU = 1 };
enum SchedMode : int32_t {
  SCHED_NATURAL = 0,   // grouped raster over the whole tile grid
  SCHED_SEGMENT = 1,   // R row segments visited in seg_order (AG sources / RS owners)
  SCHED_STRIDED = 2,   // tile owner = linear id % R, owners visited in seg_order (AR2)
  SCHED_LIST = 3,      // explicit list of row-major tile ids (repair of flagged tiles)
};

// Epilogue staging: 128 accumulator rows x 128 columns of 16-bit data. Used either as two
// 128 x 64 boxes in the layout a 128-byte-swizzled TMA store expects, or as one padded row per
// accumulator row (256 data bytes at a pitch of 272 bytes, so that the 16-byte stores of 8
// consecutive rows hit different banks while every row stays contiguous for a bulk copy).
constexpr int kStageCols = 128;
constexpr int kStageRowBytes = kStageCols * 2;
constexpr int kStagePitch = kStageRowBytes + 16;
constexpr int kStagingBytes = BM * kStagePitch;
constexpr int kBoxBytes = BM * 128;      // one 128-row x 64-column box

template <int BN, int kCtaM, bool kStaging, int kMT>
struct TileShape {
  // kCtaM = 2: two CTAs (one cluster) share each tcgen05 MMA; every CTA loads its own rows of A
  // and its own BN/2 rows of B. kMT = 2: 256 rows of A per CTA and stage.
  static_assert(kMT == 1 || (kCtaM == 2 && kStaging), "256-row CTA tiles run on CTA pairs with staging");
  static constexpr int kABytes = kMT * BM * BK * 2;
  static constexpr int kBBytes = (BN / kCtaM) * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // 227 KB per CTA: the epilogue staging is carved out for the operators whose epilogue
  // publishes tiles to other ranks and for the staged TMA-store epilogue; the others get a
  // deeper ring instead.
  static constexpr int kStagingUsed = kStaging ? kStagingBytes : 0;
  static constexpr int kStages = (226 * 1024 - kStagingUsed) / kStageBytes;
  static constexpr int kTmemCols = 2 * BN;
  // ring + epilogue staging + 1 KB for barriers and the TMEM slot; the dynamic shared array is
  // declared 1024-byte aligned
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingUsed + 1024;
};

// Per-CTA stall accounting slots (nanoseconds unless noted).
enum ProfSlot : int {
  PROF_LOAD_FLAG_WAIT = 0,   // TMA warp: waiting for all-gather tickets
  PROF_LOAD_EMPTY_WAIT = 1,  // TMA warp: waiting for a free smem stage
  PROF_MMA_FULL_WAIT = 2,    // MMA warp: waiting for operands (starved)
  PROF_MMA_TMEM_WAIT = 3,    // MMA warp: waiting for the epilogue to drain an accumulator
  PROF_EPI_BUSY = 4,         // epilogue: accumulator ready -> accumulator released
  PROF_EPI_PUBLISH = 5,      // epilogue: phase 1 (ship partials, wait for the writes, ticket)
  PROF_EPI_TICKET_WAIT = 6,  // epilogue: phase 2 (waiting for other ranks' partials)
  PROF_EPI_TILES = 7,        // epilogue: 128-row accumulators processed (count)
  PROF_PUSH_TOTAL = 8,       // communication warps: whole push / collect loop
  PROF_KERNEL = 9,           // CTA lifetime
  PROF_AR_A_WAIT = 10,       // two-shot all-reduce, owner side: waiting for the R partials of owned tiles
  PROF_AR_A_WORK = 11,       // owner side: reduce + broadcast + fence + result tickets
  PROF_AR_B_WAIT = 12,       // collector side: waiting for result tickets
  PROF_AR_B_COPY = 13,       // collector side: result buffer -> c
  PROF_EPI_DONE_AT = 14,     // kernel start -> last tile left the epilogue
  PROF_AR_A_DONE_AT = 15,    // kernel start -> last owned tile broadcast
  // time stamps (ns since this CTA started) of the LAST tile each role handled
  PROF_TL_ACC_READY = 16,    // epilogue: accumulator ready
  PROF_TL_STAGED = 17,       // epilogue: partial converted, all bulk stores issued
  PROF_TL_STORED = 18,       // epilogue: bulk stores complete
  PROF_TL_FLAGGED = 19,      // epilogue: tile ticket(s) released
  PROF_TL_OWN_SEEN = 20,     // owner: all R partial tickets seen
  PROF_TL_OWN_LOADED = 21,   // owner: reduce / broadcast loop done
  PROF_TL_OWN_FENCED = 22,   // owner: system fence + barrier passed
  PROF_TL_OWN_FLAGGED = 23,  // owner: result tickets released
  PROF_TL_COL_SEEN = 24,     // collector: last result ticket seen
  PROF_TL_COMM_START = 25,   // communication warps: entry
  PROF_TL_OWN_IT0 = 26,      // owner: first batch of the reduce loop stored (cold-start cost)
  PROF_SK_WAIT = 27,         // epilogue: split-K finisher waiting for the other slices' partials
  PROF_T_ENTRY = 28,         // absolute globaltimer: first instruction of the CTA
  PROF_T_SETUP = 29,         // absolute globaltimer: barriers initialised, TMEM allocated, roles start
  PROF_T_END = 30,           // absolute globaltimer: CTA done
  kProfSlots = 32,
};

struct alignas(64) GemmParams {
  CUtensorMap tma_a;       // A [rows, K]; for OP_AG this rank's local shard [M_pr, K]
  CUtensorMap tma_a_ws;    // OP_AG: gathered workspace [M, K] (this round's parity)
  CUtensorMap tma_b;       // B [N_rows, K], box 128 rows
  CUtensorMap tma_c32;     // local output (store map, box 32 rows x 64 columns), valid if c_tma
  // Store maps (box 128 rows x 64 columns, 128-byte swizzle) over this rank's slot inside
  // every rank's slot buffer.
  CUtensorMap tma_slot[kMaxRanks];

  int32_t M, N, K;         // output is M x N (for EPI_SWIGLU: M x N with B holding 2N rows)
  int32_t m_tiles, n_tiles, k_blocks;
  int32_t rank, R;
  int32_t op, epi, sched;
  int32_t cta_m;           // CTAs per scheduling unit along M (1, or 2 for CTA pairs)
  int32_t cta_mt;          // 128-row blocks per CTA tile (1 or 2)
  int32_t sub_tiles;       // 128-row blocks per scheduling unit = cta_m * cta_mt
  int32_t unit_m;          // scheduling units along M = ceil(m_tiles / sub_tiles)
  int32_t seg_m_tiles;     // units per segment (SCHED_SEGMENT)
  int32_t raster_g;        // units along M walked together (L2 residency of their A rows)
  int32_t seg_order[kMaxRanks];
  int32_t strided_interleave;  // SCHED_STRIDED: same unit order on every rank (see tile_at)
  int32_t seg_interleave;      // SCHED_SEGMENT: position i is tile i / R of segment order[i % R]
  const int32_t* order_table;  // optional device table overriding seg_order (R entries)
  // order_table is the order[] part of a full skew table [seq, degraded, mode, k_eff, order[R],
  // budget[R]] (reference layout, ag_tr_pred.py:14-30): the four header words stand in front of
  // it and R spin budgets behind it, and the kernel honours all of them (see the kernel prologue)
  int32_t table_has_header;
  int32_t seg_bands;           // SCHED_SEGMENT: row bands per segment walked band-major (1 = source-major)
  int32_t seg_own_first;       // band-major walk: the whole first segment of the order (own rows) before the bands of the others
  const int32_t* tile_list;    // SCHED_LIST: row-major tile ids
  int32_t list_len;
  int32_t m_per_rank;      // rows per rank (AG source shard / RS owner block)
  int32_t swiglu_up_row0;  // EPI_SWIGLU: row offset of the "up" half inside B
  int32_t is_bf16;
  uint32_t round;          // monotonic ticket of this call

  void* c;                 // local output (see per-op meaning in the kernel)
  int64_t ldc;
  int32_t c_tma;           // tma_c32 is valid: local tiles leave through staged TMA stores

  // ---- split-K of the remainder round ----
  int32_t sk_tiles;        // scheduling positions (the last ones) that are cut along K
  int32_t sk_slices;       // K ranges per such position (each on its own worker)
  float* sk_ws;            // [CTA slot][accumulator block][32-column chunk][8][128 threads] x 16 B
  uint32_t* sk_flags;      // [CTA slot]: epoch of the last partial parked in the slot
  uint32_t sk_epoch;       // per-launch value, never repeated on a device
  int32_t sk_slot_words;   // fp32 words per CTA slot

  // ---- OP_AG ----
  const void* a_local;             // this rank's shard (push source)
  void* peer_ws[kMaxRanks];        // workspace base (this round's parity) on every rank
  uint32_t* peer_ag_flags[kMaxRanks];  // [R][ag_flag_stride] tickets on every rank, indexed by source
  uint32_t* ag_counters;           // local [R + 1][n_chunks] part counters (row R: staging of the own shard, pull)
  uint32_t* peer_ag_arrive[kMaxRanks];  // pull: [R][ag_flag_stride] "source staged its chunk" tickets on every rank
  int32_t ag_pull;                 // 1 = pull transport (stage, arrive, pull, ready), 0 = push
  int32_t ag_mc;                   // OP_AG: the shard goes out as multimem.st through mc_part (all CTAs' comm warps)
  int32_t l2_ahead;                // k-blocks the producer asks L2 for ahead of its loads (0 = none)
  uint64_t* arrival_ns;            // optional [R] first-observed arrival stamps (skew observer)
  int32_t chunk_rows, n_chunks, push_parts;
  int32_t skip_comm;
  int32_t comm_only;
  int32_t publish_only;    // all-reduce decomposition: partial tiles are published and ticketed, nothing is reduced
  int32_t push_ctas;       // CTAs that take part in the all-gather push (0 = all)
  int32_t push_skip_rounds;  // scheduling rounds the pushing CTAs sit out

  // ---- OP_RS / OP_AR* ----
  void* peer_slots[kMaxRanks];     // slot base (this round's parity) on every rank: [R][rows][N]
  uint32_t* peer_tile_flags[kMaxRanks];  // [R][ticket_stride] tickets on every rank, indexed by source
  int64_t slot_stride;             // elements between two sources' slots
  void* peer_res[kMaxRanks];       // OP_AR2: reduced-result buffer [M][N] on every rank
  uint32_t* peer_res_flags[kMaxRanks];   // OP_AR2: [R][ticket_stride] tickets, indexed by owner
  int32_t res_is_c;                // OP_AR2: caller's c aliases peer_res[rank]; skip the copy
  // OP_AR2 through the switch: partials stay in this rank's own buffer (peer_slots[*] all name
  // it, slot_stride = 0); the owner of a tile sums the R copies with multimem.ld_reduce on
  // mc_part and writes the result into every rank's result buffer with multimem.st on mc_res.
  // OP_RS through the switch: the same, except that the owner of a tile is the rank that keeps
  // its rows and the sum is stored into that rank's c only.
  int32_t nvls;
  int32_t reduce_ctas;             // OP_RS through the switch: CTAs that reduce in the steady phase (0 = all)
  int32_t reduce_tail;             // ... and the number of last blocks that every CTA helps with
  void* mc_part;                   // multicast address of the partial buffer [M][N] (this parity)
  void* mc_res;                    // multicast address of the result buffer [M][N] (this parity)

  // Optional stall accounting: [gridDim.x][kProfSlots] nanosecond sums written at kernel end
  // (see ProfSlot); nullptr = off, no timer is read.
  uint64_t* prof;

  WaitEnv env;
  // Pipeline probes (plain GEMM only; results are meaningless): 1 = tensor-pipe ceiling, the
  // ring is filled once and every k-block re-multiplies resident stages without waiting for
  // loads; 2 = operand-feed ceiling, every stage is loaded and released without any MMA.
  int32_t probe;
  // Words between two sources' rows of the ticket planes. They are properties of the context
  // (its largest shape), not of the call: a word then belongs to one (source, index) pair for
  // the whole life of the context, whatever M the calls use.
  int32_t ticket_stride;   // tile tickets: [source][ticket_stride]
  int32_t ag_flag_stride;  // all-gather chunk tickets: [source][ag_flag_stride]
  int32_t pad_;
};

// ----------------------------------------------------------------------------
// Tile order
// ----------------------------------------------------------------------------
// A CTA tile: cta_mt consecutive 128-row blocks starting at `m_tile`, one BN-wide column
// block. `linear` is the ticket index of its first 128-row block (see tile_linear).
struct TileCoord {
  int m_tile, n_tile, linear, owner_key;
  bool valid;
};

__host__ __device__ __forceinline__ void raster_grouped(int u, int m_units, int n_tiles, int G, int& mt,
                                                        int& nt) {
  // Groups of G row units walked column by column: a wave of CTAs shares few A
  // row blocks and a contiguous run of B column blocks in L2.
  const int per_group = G * n_tiles;
  const int g = u / per_group;
  const int first_m = g * G;
  const int gm = min(G, m_units - first_m);
  const int r = u - g * per_group;
  mt = first_m + r % gm;
  nt = r / gm;
}

// The schedule enumerates *units*: one unit is one BN-wide column block of sub_tiles
// consecutive 128-row blocks (CTA `sub` of a pair owns blocks unit_m * sub_tiles + sub * cta_mt
// ...). `owner_key` is the unit id that decides the owning rank in the strided (two-shot
// all-reduce) order.
// `bands` > 1 (SCHED_SEGMENT): the segments are cut into that many row bands and the walk is
// band-major (band 0 of every segment in `order`, then band 1 ...) instead of source-major.
__host__ __device__ __forceinline__ TileCoord tile_at(const GemmParams& p, const int32_t* order, int pos,
                                             int sub, int bands = 1) {
  TileCoord t;
  t.valid = true;
  int um = 0, nt = 0, ulin = -1;
  if (p.sched == SCHED_SEGMENT && bands > 1 && !p.seg_interleave && p.seg_m_tiles % bands == 0) {
    const int band_units = p.seg_m_tiles / bands;
    const int per_band = band_units * p.n_tiles;
    const int per_seg = p.seg_m_tiles * p.n_tiles;
    if (p.seg_own_first && p.R > 1) {
      // the first segment of the order (this rank's own rows, which need no transfer) whole, then
      // band b of all other sources before band b + 1 of any: the order in which a transfer
      // that sends every source's rows at the same rate (multicast) completes them
      if (pos < per_seg) {
        raster_grouped(pos, p.seg_m_tiles, p.n_tiles, p.raster_g, um, nt);
        um += order[0] * p.seg_m_tiles;
      } else {
        // band b of all other sources is ONE raster area of (R - 1) * band_units row units, walked
        // in groups column by column like any other area: concurrent tiles share their B column
        // blocks (a walk source by source inside the band would stream all of B once per row unit)
        const int q = pos - per_seg;
        const int area_units = (p.R - 1) * band_units;
        const int b = q / (area_units * p.n_tiles);
        const int u = q - b * (area_units * p.n_tiles);
        int ux = 0;
        raster_grouped(u, area_units, p.n_tiles, p.raster_g, ux, nt);
        const int si = 1 + ux / band_units;
        um = order[si] * p.seg_m_tiles + b * band_units + (ux - (si - 1) * band_units);
      }
    } else {
      const int b = pos / (p.R * per_band);
      const int rem = pos - b * (p.R * per_band);
      const int si = rem / per_band;
      const int u = rem - si * per_band;
      raster_grouped(u, band_units, p.n_tiles, p.raster_g, um, nt);
      um += order[si] * p.seg_m_tiles + b * band_units;
    }
  } else if (p.sched == SCHED_SEGMENT) {
    const int per_seg = p.seg_m_tiles * p.n_tiles;
    // interleaved: every rank walks the segments in lockstep (tile k of every owner, then tile
    // k + 1 ...), so that all partials of a tile exist at about the same time on all ranks
    const int si = p.seg_interleave ? pos % p.R : pos / per_seg;
    const int u = p.seg_interleave ? pos / p.R : pos - si * per_seg;
    raster_grouped(u, p.seg_m_tiles, p.n_tiles, p.raster_g, um, nt);
    um += order[si] * p.seg_m_tiles;
  } else if (p.sched == SCHED_STRIDED) {
    const int total = p.unit_m * p.n_tiles;
    const int per_owner = (total + p.R - 1) / p.R;
    const int oi = pos / per_owner;
    const int k = pos - oi * per_owner;
    // interleaved: every rank walks the units in the same order, so the partials of a unit
    // reach its owner while the owner computes its own, and the owners' broadcasts spread
    // over the whole kernel instead of piling up at the end
    ulin = p.strided_interleave ? pos : order[oi] + k * p.R;
    if (ulin >= total) t.valid = false;
    else raster_grouped(ulin, p.unit_m, p.n_tiles, p.raster_g, um, nt);
  } else if (p.sched == SCHED_LIST) {
    const int lin = p.tile_list[pos];
    t.valid = lin >= 0 && lin < p.unit_m * p.n_tiles;
    um = t.valid ? lin / p.n_tiles : 0;
    nt = t.valid ? lin - um * p.n_tiles : 0;
  } else {
    raster_grouped(pos, p.unit_m, p.n_tiles, p.raster_g, um, nt);
  }
  t.m_tile = um * p.sub_tiles + sub * p.cta_mt;
  t.n_tile = nt;
  t.owner_key = ulin;
  // ownership is keyed by the pre-raster unit id; every 128-row block still has its own ticket
  t.linear = (p.sched == SCHED_STRIDED) ? ulin * p.sub_tiles + sub * p.cta_mt : t.m_tile * p.n_tiles + nt;
  return t;
}

// Ticket index of the h-th 128-row block of a CTA tile.
__host__ __device__ __forceinline__ int tile_linear(const GemmParams& p, const TileCoord& t, int h) {
  return (p.sched == SCHED_STRIDED) ? t.linear + h : t.linear + h * p.n_tiles;
}

__host__ __device__ __forceinline__ int sched_positions(const GemmParams& p) {
  const int total = p.unit_m * p.n_tiles;
  if (p.sched == SCHED_STRIDED) return ((total + p.R - 1) / p.R) * p.R;
  if (p.sched == SCHED_LIST) return p.list_len;
  return total;
}

// Static round-robin of the scheduling positions over the workers (a worker is a CTA, or a CTA
// pair), with two twists. The workers that push the all-gather shard sit out the first `skip`
// rounds (their copy engine is busy and their operand loads are slower meanwhile), so that all
// workers finish together. And the positions of the last, partial round (`sk_tiles` of them)
// are not dealt whole: each is cut into `sk_slices` K ranges, dealt to consecutive workers.
// Shared by the kernel and the host-side schedule dump.
struct WorkerSchedule {
  int workers;   // workers in the grid
  int pushers;   // workers 0 .. pushers-1 drive the all-gather push
  int skip;      // rounds the pushers sit out
  int early;     // workers active in the early rounds
  int dp_positions;   // positions dealt whole
  int sk_tiles, sk_slices;
  __host__ __device__ int pos_of(int my_worker, int i) const {
    if (my_worker < pushers) return skip * early + i * workers + my_worker;
    if (i < skip) return i * early + (my_worker - pushers);
    return skip * early + (i - skip) * workers + my_worker;
  }
};
__host__ __device__ __forceinline__ WorkerSchedule make_worker_schedule(const GemmParams& p, int grid_x,
                                                                        int cta_m) {
  WorkerSchedule w;
  w.workers = grid_x / cta_m;
  w.pushers = 0;
  w.skip = 0;
  if (p.op == OP_AG && p.R > 1 && !p.skip_comm && p.push_ctas > 0 && p.push_ctas < grid_x) {
    w.pushers = (p.push_ctas + cta_m - 1) / cta_m;
    w.skip = p.push_skip_rounds;
  }
  w.early = w.workers - w.pushers;
  const int positions = p.comm_only ? 0 : sched_positions(p);
  w.sk_tiles = (p.sk_slices > 1 && p.sk_tiles <= positions) ? p.sk_tiles : 0;
  w.sk_slices = w.sk_tiles > 0 ? p.sk_slices : 1;
  w.dp_positions = positions - w.sk_tiles;
  return w;
}

// How many of the `positions` fall into the last, partial round of the round-robin (0 = the
// rounds come out even), for a grid of `workers` workers of which `pushers` skip `skip` rounds.
__host__ __device__ __forceinline__ int remainder_positions(int positions, int workers, int pushers, int skip) {
  const int early = workers - pushers;
  const int head = skip * early;
  if (positions <= head) return 0;
  return (positions - head) % workers;
}

// One piece of work of a worker: scheduling position `pos`, k-blocks [kb0, kb1). slices > 1:
// the position is shared with slices - 1 other workers; slice 0 finishes the tile.
struct WorkItem {
  int pos, kb0, kb1, slice, slices;
};
struct WorkIter {
  int i = 0;
  bool sk_seen = false;
  __host__ __device__ bool next(const WorkerSchedule& w, int my_worker, int k_blocks, WorkItem& wi) {
    if (sk_seen) return false;
    const int pos = w.pos_of(my_worker, i);
    if (pos < w.dp_positions) {
      ++i;
      wi.pos = pos; wi.kb0 = 0; wi.kb1 = k_blocks; wi.slice = 0; wi.slices = 1;
      return true;
    }
    sk_seen = true;
    if (my_worker >= w.sk_tiles * w.sk_slices) return false;
    const int t = my_worker / w.sk_slices, s = my_worker - t * w.sk_slices;
    wi.pos = w.dp_positions + t;
    wi.kb0 = static_cast<int>(static_cast<long long>(s) * k_blocks / w.sk_slices);
    wi.kb1 = static_cast<int>(static_cast<long long>(s + 1) * k_blocks / w.sk_slices);
    wi.slice = s;
    wi.slices = w.sk_slices;
    return true;
  }
};

// ----------------------------------------------------------------------------
// Epilogue helpers
// ----------------------------------------------------------------------------
template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (kBf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}
template <bool kBf16>
__device__ __forceinline__ float2 unpack2(uint32_t u) {
  if constexpr (kBf16) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  } else {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
}

// Adds 32 consecutive 16-bit values at `src` (64 bytes, not cached in L1) to acc.
template <bool kBf16>
__device__ __forceinline__ void add_row32(float (&acc)[32], const void* src) {
  const uint4* s = reinterpret_cast<const uint4*>(src);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint4 v = ld_global_cg_v4(s + q);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack2<kBf16>(w[j]);
      acc[q * 8 + j * 2] += f.x;
      acc[q * 8 + j * 2 + 1] += f.y;
    }
  }
}

// acc += sum over sources s in [0, R), s != skip, of the 32 16-bit values at
// base + s * stride_bytes (64 bytes each). Loads of four sources are issued together so
// that their latencies overlap; the accumulation order is fixed (ascending s).
template <bool kBf16>
__device__ __forceinline__ void add_rows32_from_sources(float (&acc)[32], const uint8_t* base,
                                                        int64_t stride_bytes, int R, int skip) {
  constexpr int kBatch = 3;
  for (int s0 = 0; s0 < R; s0 += kBatch) {
    uint4 v[kBatch][4];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int s = s0 + u;
      const bool on = s < R && s != skip;
      const uint4* src = reinterpret_cast<const uint4*>(base + (on ? s : 0) * stride_bytes);
#pragma unroll
      for (int q = 0; q < 4; ++q) v[u][q] = on ? ld_global_cg_v4(src + q) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t w[4] = {v[u][q].x, v[u][q].y, v[u][q].z, v[u][q].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack2<kBf16>(w[j]);   // inactive sources contribute +0.0
          acc[q * 8 + j * 2] += f.x;
          acc[q * 8 + j * 2 + 1] += f.y;
        }
      }
    }
  }
}

// Stores the first `cols` (a multiple of 8, at most 32) of 32 consecutive values of a row.
template <bool kBf16>
__device__ __forceinline__ void store_row32(void* dst, const float (&acc)[32], int cols = 32) {
  uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    if (q * 8 >= cols) break;
    uint4 v;
    v.x = pack2<kBf16>(acc[q * 8 + 0], acc[q * 8 + 1]);
    v.y = pack2<kBf16>(acc[q * 8 + 2], acc[q * 8 + 3]);
    v.z = pack2<kBf16>(acc[q * 8 + 4], acc[q * 8 + 5]);
    v.w = pack2<kBf16>(acc[q * 8 + 6], acc[q * 8 + 7]);
    st_global_v4(d + q, v);
  }
}

// Rounds the accumulator through the 16-bit output type (so that a value every
// rank re-derives from the same 16-bit partials is bit-identical everywhere).
template <bool kBf16>
__device__ __forceinline__ void round_row32(float (&acc)[32]) {
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float2 f = unpack2<kBf16>(pack2<kBf16>(acc[2 * j], acc[2 * j + 1]));
    acc[2 * j] = f.x;
    acc[2 * j + 1] = f.y;
  }
}

// Epilogue staging in the layout a 128-byte-swizzled TMA store expects: two boxes of
// [128 rows x 64 columns]; inside a box row r occupies 128 bytes and its 16-byte chunk c
// sits at chunk position c ^ (r & 7). `cc` selects the 32-column quarter of the 128 staged
// columns.
template <bool kBf16>
__device__ __forceinline__ void stage_row32_swizzled(uint8_t* staging, int r, int cc, const float (&acc)[32]) {
  uint8_t* box_row = staging + (cc >> 1) * (BM * 128) + r * 128;
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    uint4 o;
    o.x = pack2<kBf16>(acc[v * 8 + 0], acc[v * 8 + 1]);
    o.y = pack2<kBf16>(acc[v * 8 + 2], acc[v * 8 + 3]);
    o.z = pack2<kBf16>(acc[v * 8 + 4], acc[v * 8 + 5]);
    o.w = pack2<kBf16>(acc[v * 8 + 6], acc[v * 8 + 7]);
    const int chunk = ((cc & 1) * 4 + v) ^ (r & 7);
    *reinterpret_cast<uint4*>(box_row + chunk * 16) = o;
  }
}

// Collective decision of the four epilogue warps. The flag is sticky; the
// second barrier keeps a fast warp from raising it for a later check while a
// slow warp has not read it yet, so all 128 threads always agree. flags[3] carries a
// value that thread 0 of the group wrote before the call (read by all between the barriers).
__device__ __forceinline__ bool epi_vote(volatile int32_t* flags, bool my_ok, int32_t* carried = nullptr) {
  if (!my_ok) flags[0] = 1;
  named_bar_sync(2, kEpiThreads);
  const bool dead = flags[0] != 0;
  if (carried) *carried = flags[3];
  named_bar_sync(2, kEpiThreads);
  return !dead;
}

__device__ __forceinline__ float silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// ----------------------------------------------------------------------------
// The kernel
// ----------------------------------------------------------------------------
template <int BN, bool kBf16, int kCtaM, bool kStaging, int kMT>
// 320 threads are allocated as 12 warps' worth of registers: 65536 / 384 = 170, so 168 per thread
// is all one CTA can have (a larger cap leaves no CTA resident at all).
__global__ void __launch_bounds__(kThreads, 1)
fused_gemm_kernel(const __grid_constant__ GemmParams p0, const GemmParams* __restrict__ pv) {
  using TS = TileShape<BN, kCtaM, kStaging, kMT>;
  static_assert(kCtaM == 1 || BN == 256, "CTA pairs are built for 256-wide tiles only");
  // With pv != nullptr the launch emulates several ranks on one GPU: grid.y
  // indexes the rank and each rank reads its own parameter block.
  const GemmParams& p = pv ? pv[blockIdx.y] : p0;

  const uint64_t t_entry = p.prof ? globaltimer_ns() : 0;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* ring = smem;
  uint8_t* staging = smem + TS::kStages * TS::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + TS::kStagingUsed);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + TS::kStages;
  uint64_t* tmem_full_bar = bars + 2 * TS::kStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint64_t* drain_bar = tmem_empty_bar + 2;
  uint64_t* push_bar = drain_bar + 1;            // barriers of the all-gather push ring
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(push_bar + kPushSlots);
  int32_t* s_order = reinterpret_cast<int32_t*>(tmem_slot + 4);
  int32_t* s_budget = s_order + kMaxRanks;   // spin budget per source (skew table)
  int32_t* s_tab = s_budget + kMaxRanks;     // [0]: row bands of the segment walk
  // s_flags[0]: an epilogue warp gave up; [1]: outcome of the comm warps' last wait; [2]: the
  // all-gather push of this CTA no longer uses the staging area; [3]: the epilogue's copy of [2]
  volatile int32_t* s_flags = s_tab + 4;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // CTA pair: rank 0 of the cluster is the leader (issues the MMAs, owns the full and
  // TMEM-empty barriers the pair synchronises on).
  const int sub = (kCtaM == 2) ? static_cast<int>(cluster_ctarank()) : 0;
  const bool leader = sub == 0;
  const WorkerSchedule wsched = make_worker_schedule(p, static_cast<int>(gridDim.x), kCtaM);
  const int my_worker = static_cast<int>(blockIdx.x) / kCtaM;
  const int push_grid = (p.push_ctas > 0 && p.push_ctas < static_cast<int>(gridDim.x))
                            ? p.push_ctas : static_cast<int>(gridDim.x);
  const bool pushes = kStaging && p.op == OP_AG && p.R > 1 && !p.skip_comm &&
                      static_cast<int>(blockIdx.x) < push_grid;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TS::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], 4 * kCtaM);
    }
    mbar_init(drain_bar, 1);
    for (int i = 0; i < kPushSlots; ++i) mbar_init(&push_bar[i], 1);
    s_flags[0] = 0;
    s_flags[1] = 1;
    s_flags[2] = pushes ? 0 : 1;   // a CTA that carries the transfer computes nothing until its part is out
    s_flags[3] = 0;
    mbar_fence_init();
  }
  if (threadIdx.x < kMaxRanks) {
    // The skew table of this call: [seq, degraded, mode, k_eff | order[R] | budget[R]].
    //   degraded = 1  the predictor stepped back: default rotation, band-major
    //   mode = 0      band-major walk (k_eff row bands per source) in the table's order
    //   mode = 1      source-major walk in the table's order (predicted-early sources first)
    //   budget[s]     polls of source s's ticket between two looks at the abort word and the clock
    const int i = threadIdx.x;
    const bool full = p.order_table != nullptr && p.table_has_header;
    const bool degraded = full && p.order_table[-3] != 0;
    s_order[i] = (p.order_table != nullptr && i < p.R && !degraded) ? p.order_table[i] : p.seg_order[i];
    s_budget[i] = (full && i < p.R) ? max(1, p.order_table[p.R + i]) : 64;
    if (i == 0) {
      int bands = p.seg_bands > 0 ? p.seg_bands : 1;
      if (full) {
        const int mode = p.order_table[-2], k_eff = p.order_table[-1];
        bands = (mode == 1 && !degraded) ? 1 : max(1, min(k_eff, p.n_chunks));
      }
      if (p.sched != SCHED_SEGMENT || p.seg_m_tiles % bands != 0) bands = 1;
      s_tab[0] = bands;
    }
  }
  if (warp == 1) {
    if constexpr (kCtaM == 2) {
      tmem_alloc_pair(tmem_slot, TS::kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, TS::kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  if constexpr (kCtaM == 2) cluster_sync_all();   // the peer's barriers are initialised too
  else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const int bands = *reinterpret_cast<volatile int32_t*>(s_tab);

  // a reference into the parameter block: a local copy would be indexed dynamically
  // (peer_abort[i]) and live on the stack, and every wait would read it from there
  const WaitEnv& env = p.env;
  uint64_t* const prof = p.prof ? p.prof + static_cast<int64_t>(blockIdx.x) * kProfSlots : nullptr;
  const uint64_t t_kernel0 = prof ? globaltimer_ns() : 0;

  // ==========================================================================
  // warp 0: TMA producer
  // ==========================================================================
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&p.tma_a);
      tma_prefetch_desc(&p.tma_b);
      if (p.op == OP_AG) tma_prefetch_desc(&p.tma_a_ws);
      uint32_t stage = 0, phase = 0;
      uint64_t acc_a = 0, acc_b = 0;
      uint32_t ready_mask[kMaxRanks] = {0};   // chunks of each source already observed
      uint32_t pending = 0;                   // stages with a load in flight (bitmask)
      int loads_issued = 0;
      bool ok = true;
      // Everything the k-block loop needs lives in registers: the inline-asm statements below
      // clobber memory, so a field read through `p` inside the loop would be re-loaded on
      // every k-block, in the one thread whose latency paces the whole operand pipeline.
      const int k_blocks = p.k_blocks;
      const int probe = p.probe;
      const bool swiglu = p.epi == EPI_SWIGLU;
      const int up_row0 = p.swiglu_up_row0;
      const CUtensorMap* const bmap = &p.tma_b;
      const int ahead = p.l2_ahead;
      if (pushes) {
        // the operand ring carries this CTA's part of the all-gather push first (the multicast
        // form leaves the ring alone, but its loads and stores would starve this SM's operand
        // feed just the same: the sending CTAs sit the transfer out as well) (the pushing
        // thread's own waits are bounded, so this one ends too; the limit is a backstop)
        const uint64_t t0 = globaltimer_ns();
        while (s_flags[2] == 0) {
          __nanosleep(200);
          if (globaltimer_ns() - t0 > 2 * env.timeout_ns) { ok = false; break; }
        }
        fence_proxy_async_smem();
      }
      WorkIter wit;
      WorkItem wi;
      while (ok && wit.next(wsched, my_worker, k_blocks, wi)) {
        const TileCoord t = tile_at(p, s_order, wi.pos, sub, bands);
        if (!t.valid) continue;
        const int m0 = t.m_tile * BM;          // first of the CTA tile's kMT * 128 rows
        const int n0 = t.n_tile * BN;
        const CUtensorMap* amap = &p.tma_a;
        int a_row = m0;
        if (p.op == OP_AG) {
          const int src = m0 / p.m_per_rank;
          if (src == p.rank) {
            a_row = m0 - p.rank * p.m_per_rank;
          } else {
            amap = &p.tma_a_ws;
            if (!p.skip_comm) {
              // every chunk the CTA tile's rows touch must have landed
              const int r_lo = m0 - src * p.m_per_rank;
              const int r_hi = min(r_lo + kMT * BM, p.m_per_rank) - 1;
              for (int ck = r_lo / p.chunk_rows; ok && ck <= r_hi / p.chunk_rows; ++ck) {
                if (ck < 32 && (ready_mask[src] >> ck) & 1u) continue;
                if (src < 0 || src >= p.R || ck >= p.ag_flag_stride) {     // never index a ticket plane blindly
                  report_failure(env, ST_BAD_INDEX, SITE_INDEX_CHECK, static_cast<uint32_t>(p.ag_flag_stride),
                                 static_cast<uint32_t>(ck), static_cast<uint32_t>(src));
                  ok = false;
                  break;
                }
                const uint32_t* f = p.peer_ag_flags[p.rank] + src * p.ag_flag_stride + ck;
                const uint64_t tw = prof ? globaltimer_ns() : 0;
                ok = wait_flag_ge(f, p.round, env, SITE_AG_CHUNK, (src << 16) | ck,
                                  static_cast<uint32_t>(s_budget[src]));
                if (prof) acc_a += globaltimer_ns() - tw;
                if (ok) {
                  if (ck < 32) ready_mask[src] |= 1u << ck;
                  if (p.arrival_ns != nullptr && ck == 0)
                    atomicMin(reinterpret_cast<unsigned long long*>(p.arrival_ns + src),
                              static_cast<unsigned long long>(globaltimer_ns()));
                }
              }
              if (!ok) break;
              // remote generic-proxy stores observed through the acquire above are
              // ordered before the async-proxy (TMA) reads below
              fence_proxy_async_all();
            }
          }
        }
        const int b_row_pair = swiglu
            ? (sub == 0 ? t.n_tile * (BN / 2) : up_row0 + t.n_tile * (BN / 2))
            : n0 + sub * (BN / 2);
        // L2 look-ahead: the ring holds about a microsecond of operands, less than a DRAM access
        // under load, so a tile whose operands are not in L2 yet (a cold start, a new column
        // block of B) would run at DRAM latency. The box `ahead` k-blocks on is requested now;
        // at the start of a tile the first `ahead` boxes are requested in one go.
        const int b_row_pf = (kCtaM == 2) ? b_row_pair : (swiglu ? t.n_tile * (BN / 2) : n0);
        const int b_row_pf2 = swiglu ? up_row0 + t.n_tile * (BN / 2) : n0 + 128;
        auto l2_request = [&](int kb) {
#pragma unroll
          for (int h = 0; h < kMT; ++h) tma_prefetch_l2_2d(amap, kb * BK, a_row + h * BM);
          tma_prefetch_l2_2d(bmap, kb * BK, b_row_pf);
          if (kCtaM == 1 && BN == 256) tma_prefetch_l2_2d(bmap, kb * BK, b_row_pf2);
        };
        if (ahead > 0 && probe == 0)
          for (int kb = wi.kb0 + 1; kb < wi.kb1 && kb < wi.kb0 + ahead; ++kb) l2_request(kb);
        for (int kb = wi.kb0; kb < wi.kb1; ++kb) {
          if (probe == 1) {
            if (loads_issued >= TS::kStages) break;   // ring filled once, then idle
            ++loads_issued;
          }
          if (ahead > 0 && kb + ahead < wi.kb1 && probe == 0) l2_request(kb + ahead);
          if (prof && !mbar_try_wait(&empty_bar[stage], phase ^ 1u)) {
            const uint64_t tw = globaltimer_ns();
            ok = wait_mbar(&empty_bar[stage], phase ^ 1u, env, SITE_PIPE_EMPTY, stage);
            acc_b += globaltimer_ns() - tw;
          } else {
            ok = wait_mbar(&empty_bar[stage], phase ^ 1u, env, SITE_PIPE_EMPTY, stage);
          }
          if (!ok) break;
          pending &= ~(1u << stage);
          uint8_t* sa = ring + stage * TS::kStageBytes;
          uint8_t* sb = sa + TS::kABytes;
          if constexpr (kCtaM == 2) {
            // the leader's barrier collects the bytes of both CTAs' loads
            if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * TS::kStageBytes);
#pragma unroll
            for (int h = 0; h < kMT; ++h)
              tma_load_2d_pair(sa + h * (BM * BK * 2), amap, &full_bar[stage], kb * BK, a_row + h * BM);
            tma_load_2d_pair(sb, bmap, &full_bar[stage], kb * BK, b_row_pair);
          } else {
            mbar_arrive_expect_tx(&full_bar[stage], TS::kStageBytes);
            tma_load_2d(sa, amap, &full_bar[stage], kb * BK, a_row);
            if (swiglu) {
              // gate rows and the matching up rows form one BN-wide virtual tile
              tma_load_2d(sb, bmap, &full_bar[stage], kb * BK, t.n_tile * (BN / 2));
              tma_load_2d(sb + (BN / 2) * BK * 2, bmap, &full_bar[stage], kb * BK,
                          up_row0 + t.n_tile * (BN / 2));
            } else {
#pragma unroll
              for (int h = 0; h < BN / 128; ++h)
                tma_load_2d(sb + h * 128 * BK * 2, bmap, &full_bar[stage], kb * BK, n0 + h * 128);
            }
          }
          pending |= 1u << stage;
          if (++stage == TS::kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (prof) {
        prof[PROF_LOAD_FLAG_WAIT] = acc_a;
        prof[PROF_LOAD_EMPTY_WAIT] = acc_b;
      }
      if (!ok) {
        // Unwinding: let the loads already issued land before the CTA's shared
        // memory is released (each such wait is itself bounded).
        for (int s = 0; s < TS::kStages; ++s) {
          if (!((pending >> s) & 1u)) continue;
          // the stage was armed in the most recent pass over slot s
          const uint32_t par = (s < static_cast<int>(stage)) ? phase : (phase ^ 1u);
          WaitEnv quiet{};                 // no status, no abort words: this wait only drains
          quiet.rank = env.rank;
          quiet.timeout_ns = 2000000ull;   // loads land within microseconds; never linger here
          if (leader) wait_mbar(&full_bar[s], par, quiet, SITE_PIPE_FULL, s);
        }
      }
    }
  }
  // ==========================================================================
  // warp 1: MMA issuer
  // ==========================================================================
  else if (warp == 1) {
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = umma_idesc_f16(kBf16, BM * kCtaM, BN);
      uint32_t stage = 0, phase = 0;
      uint64_t acc_f = 0, acc_t = 0;
      int it = 0;
      int kblocks_done = 0;
      bool ok = true;
      // registers only inside the k-block loop (see the producer warp); the operand descriptors
      // of stage s are those of stage 0 plus s times the stage size in 16-byte units
      const int k_blocks = p.k_blocks;
      const int probe = p.probe;
      const uint64_t da0 = umma_desc_k_sw128(smem_u32(ring));
      const uint64_t db0 = umma_desc_k_sw128(smem_u32(ring) + TS::kABytes);
      constexpr uint64_t kDescStage = static_cast<uint64_t>(TS::kStageBytes >> 4);
      constexpr uint64_t kDescRows = static_cast<uint64_t>((BM * BK * 2) >> 4);   // next 128 rows of A
      // four MMAs of one 64-wide k-block into accumulator d_tmem; `fresh` overwrites it
      auto mma4 = [&](uint32_t d_tmem, uint64_t da, uint64_t db, bool fresh) {
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          // +32 bytes per K step inside the 128-byte swizzle row
          if constexpr (kCtaM == 2)
            umma_f16_ss_pair(d_tmem, da + static_cast<uint64_t>(k * 2), db + static_cast<uint64_t>(k * 2),
                             idesc, (fresh && k == 0) ? 0u : 1u);
          else
            umma_f16_ss(d_tmem, da + static_cast<uint64_t>(k * 2), db + static_cast<uint64_t>(k * 2), idesc,
                        (fresh && k == 0) ? 0u : 1u);
        }
      };
      // frees the smem stage (in both CTAs of a pair) when the MMAs issued so far retire
      auto commit_stage = [&](uint32_t s) {
        if constexpr (kCtaM == 2) umma_commit_pair_both(&empty_bar[s]);
        else umma_commit(&empty_bar[s]);
      };
      // accumulator complete (each CTA of a pair reads its own 128 rows)
      auto commit_acc = [&](int b) {
        if constexpr (kCtaM == 2) umma_commit_pair_both(&tmem_full_bar[b]);
        else umma_commit(&tmem_full_bar[b]);
      };
      auto wait_full = [&](uint32_t s, uint32_t ph) -> bool {
        if (mbar_try_wait(&full_bar[s], ph)) return true;
        const uint64_t tw = prof ? globaltimer_ns() : 0;
        const bool r = wait_mbar(&full_bar[s], ph, env, SITE_PIPE_FULL, s);
        if (prof) acc_f += globaltimer_ns() - tw;
        return r;
      };
      auto wait_acc_free = [&](int b, uint32_t par) -> bool {
        if (mbar_try_wait(&tmem_empty_bar[b], par)) return true;
        const uint64_t tw = prof ? globaltimer_ns() : 0;
        const bool r = wait_mbar(&tmem_empty_bar[b], par, env, SITE_TMEM_EMPTY, b);
        if (prof) acc_t += globaltimer_ns() - tw;
        return r;
      };
      WorkIter wit;
      WorkItem wi;
      while (ok && wit.next(wsched, my_worker, k_blocks, wi)) {
        const TileCoord t = tile_at(p, s_order, wi.pos, sub, bands);
        if (!t.valid) continue;
        const int nkb = wi.kb1 - wi.kb0;
        if constexpr (kMT == 1) {
          // the two accumulators double-buffer whole tiles
          const int buf = it & 1;
          const uint32_t use = static_cast<uint32_t>(it >> 1);
          ok = wait_acc_free(buf, (use & 1u) ^ 1u);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BN);
          for (int j = 0; j < nkb; ++j) {
            if (!(probe == 1 && kblocks_done >= TS::kStages)) {
              // (probe 1, tensor-pipe ceiling: stages filled in the first pass stay resident)
              ok = wait_full(stage, phase);
              if (!ok) break;
            }
            if (probe != 0) {
              ++kblocks_done;
              if (probe == 2) {
                // operand-feed ceiling: hand the stage straight back to the producer(s)
                mbar_arrive(&empty_bar[stage]);
                if constexpr (kCtaM == 2) mbar_arrive_cluster(&empty_bar[stage], 1u);
                if (++stage == TS::kStages) { stage = 0; phase ^= 1u; }
                continue;
              }
            }
            tc_fence_after_sync();
            mma4(d_tmem, da0 + stage * kDescStage, db0 + stage * kDescStage, j == 0);
            commit_stage(stage);
            if (++stage == TS::kStages) { stage = 0; phase ^= 1u; }
          }
          if (!ok) break;
          commit_acc(buf);
        } else {
          // One accumulator per 128-row half, both used by every tile. Half 0 is drained first
          // by the epilogue, so its MMAs of the first k-blocks are issued as soon as accumulator
          // 0 is free, while accumulator 1 is still being drained; the stages stay occupied
          // until half 1 has consumed them too.
          const uint32_t par_free = static_cast<uint32_t>(it & 1) ^ 1u;
          const int ahead = (probe == 1 || probe == 2) ? 0 : min(static_cast<int>(TS::kStages), nkb);
          ok = wait_acc_free(0, par_free);
          if (!ok) break;
          tc_fence_after_sync();
          uint32_t s1 = stage, ph1 = phase;
          for (int j = 0; j < ahead; ++j) {
            ok = wait_full(s1, ph1);
            if (!ok) break;
            tc_fence_after_sync();
            mma4(tmem_base, da0 + s1 * kDescStage, db0 + s1 * kDescStage, j == 0);
            if (j == nkb - 1) commit_acc(0);
            if (++s1 == TS::kStages) { s1 = 0; ph1 ^= 1u; }
          }
          if (!ok) break;
          ok = wait_acc_free(1, par_free);
          if (!ok) break;
          tc_fence_after_sync();
          for (int j = 0; j < ahead; ++j) {
            mma4(tmem_base + BN, da0 + stage * kDescStage + kDescRows, db0 + stage * kDescStage, j == 0);
            commit_stage(stage);
            if (j == nkb - 1) commit_acc(1);
            if (++stage == TS::kStages) { stage = 0; phase ^= 1u; }
          }
          for (int j = ahead; j < nkb; ++j) {
            if (!(probe == 1 && kblocks_done >= TS::kStages)) {
              ok = wait_full(stage, phase);
              if (!ok) break;
            }
            if (probe != 0) {
              ++kblocks_done;
              if (probe == 2) {
                mbar_arrive(&empty_bar[stage]);
                mbar_arrive_cluster(&empty_bar[stage], 1u);
                if (j == nkb - 1) { commit_acc(0); commit_acc(1); }
                if (++stage == TS::kStages) { stage = 0; phase ^= 1u; }
                continue;
              }
            }
            tc_fence_after_sync();
            mma4(tmem_base, da0 + stage * kDescStage, db0 + stage * kDescStage, j == 0);
            if (j == nkb - 1) commit_acc(0);
            mma4(tmem_base + BN, da0 + stage * kDescStage + kDescRows, db0 + stage * kDescStage, j == 0);
            commit_stage(stage);
            if (j == nkb - 1) commit_acc(1);
            if (++stage == TS::kStages) { stage = 0; phase ^= 1u; }
          }
          if (!ok) break;
        }
        ++it;
      }
      if (prof) {
        prof[PROF_MMA_FULL_WAIT] = acc_f;
        prof[PROF_MMA_TMEM_WAIT] = acc_t;
      }
      if (!ok) {
        // Unwinding: MMAs already issued must retire before TMEM is freed.
        if constexpr (kCtaM == 2) umma_commit_pair_local(drain_bar);
        else umma_commit(drain_bar);
        WaitEnv quiet{};
        quiet.rank = env.rank;
        quiet.timeout_ns = env.timeout_ns;
        wait_mbar(drain_bar, 0u, quiet, SITE_TMEM_FULL, 0);
      }
    }
  }
  // ==========================================================================
  // warps 2-5: epilogue
  // ==========================================================================
  else if (warp < kCommWarp0) {
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int etid = (warp - kEpiWarp0) * 32 + lane;
    const int r_in_tile = q * 32 + lane;
    const int64_t ldc = p.ldc;
    const int tiles = p.ticket_stride;                  // ticket words per source
    const bool multi = p.R > 1;
    // scratch slots of the split-K partials are indexed by the CTA's place in the launch
    const int slot0 = static_cast<int>(blockIdx.y * gridDim.x);
    const int my_slot = slot0 + static_cast<int>(blockIdx.x);
    uint64_t acc_busy = 0, acc_pub = 0, acc_tick = 0, acc_sk = 0, n_tiles_done = 0;
    int it = 0;
    bool alive = true;
    WorkIter wit;
    WorkItem wi;
    while (alive && wit.next(wsched, my_worker, p.k_blocks, wi)) {
      const TileCoord t = tile_at(p, s_order, wi.pos, sub, bands);
      if (!t.valid) continue;
      for (int h = 0; alive && h < kMT; ++h) {
      const int buf = (kMT == 2) ? h : (it & 1);
      const uint32_t par = (kMT == 2) ? static_cast<uint32_t>(it & 1) : static_cast<uint32_t>((it >> 1) & 1);
      const int m_tile = t.m_tile + h;
      const int lin = tile_linear(p, t, h);
      // The four epilogue warps decide together whether to go on: a warp that
      // gave up must never leave the others parked at a named barrier.
      // one lane per warp polls (the other 31 sleep at the warp barrier): the epilogue warps
      // spend most of the kernel here, and idle polling costs power the tensor cores need
      bool acc_ready = true;
      if (lane == 0) acc_ready = wait_mbar(&tmem_full_bar[buf], par, env, SITE_TMEM_FULL, buf);
      acc_ready = __shfl_sync(0xFFFFFFFFu, acc_ready ? 1 : 0, 0) != 0;
      if (etid == 0) s_flags[3] = s_flags[2];
      int32_t stg = 0;
      if (!epi_vote(s_flags, acc_ready, &stg)) { alive = false; break; }
      const bool staging_free = kStaging && stg != 0;   // not in use by this CTA's all-gather push
      tc_fence_after_sync();
      const uint64_t t_epi0 = (prof && etid == 0) ? globaltimer_ns() : 0;
      if (prof && etid == 0) prof[PROF_TL_ACC_READY] = t_epi0 - t_kernel0;

      const int row = m_tile * BM + r_in_tile;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                             static_cast<uint32_t>(buf * BN);
      bool released = false;
      // accumulator drained: hand the TMEM buffer back to the MMA warp
      auto release_acc = [&]() {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (kCtaM == 2) mbar_arrive_leader(&tmem_empty_bar[buf]);
          else mbar_arrive(&tmem_empty_bar[buf]);
        }
        released = true;
      };

      // ---- split-K: slices other than 0 park their fp32 accumulator and are done ----------
      if (wi.slices > 1) {
        // layout of a slot: [accumulator block][32-column chunk][16-byte piece][thread]
        if (wi.slice > 0) {
          float* dst = p.sk_ws + static_cast<int64_t>(my_slot) * p.sk_slot_words + h * (BM * BN);
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int v = 0; v < 8; ++v)
              st_global_v4(dst + ((c * 8 + v) * kEpiThreads + etid) * 4,
                           make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]));
          }
          release_acc();
          if (h == kMT - 1) {
            // the barrier orders all 128 threads' stores before the one release below
            named_bar_sync(2, kEpiThreads);
            if (etid == 0) st_release_gpu(p.sk_flags + my_slot, p.sk_epoch);
          }
          if (prof && etid == 0) {
            acc_busy += globaltimer_ns() - t_epi0;
            ++n_tiles_done;
          }
          continue;
        }
        // slice 0: add the partials of slices 1 .. slices-1 (the next workers) in that order
        const uint64_t t_sk0 = (prof && etid == 0) ? globaltimer_ns() : 0;
        bool ok = true;
        if (etid == 0) {
          for (int s = 1; ok && s < wi.slices; ++s)
            ok = wait_flag_ge(p.sk_flags + slot0 + (my_worker + s) * kCtaM + sub, p.sk_epoch, env,
                              SITE_SPLITK, s);
        }
        if (!epi_vote(s_flags, ok)) { alive = false; break; }
        if (prof && etid == 0) acc_sk += globaltimer_ns() - t_sk0;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c * 32, r);
          tmem_ld_wait();
          for (int s = 1; s < wi.slices; ++s) {
            const float* src = p.sk_ws +
                static_cast<int64_t>(slot0 + (my_worker + s) * kCtaM + sub) * p.sk_slot_words + h * (BM * BN);
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              const uint4 x = ld_global_cg_v4(src + ((c * 8 + v) * kEpiThreads + etid) * 4);
              r[v * 4 + 0] = __float_as_uint(__uint_as_float(r[v * 4 + 0]) + __uint_as_float(x.x));
              r[v * 4 + 1] = __float_as_uint(__uint_as_float(r[v * 4 + 1]) + __uint_as_float(x.y));
              r[v * 4 + 2] = __float_as_uint(__uint_as_float(r[v * 4 + 2]) + __uint_as_float(x.z));
              r[v * 4 + 3] = __float_as_uint(__uint_as_float(r[v * 4 + 3]) + __uint_as_float(x.w));
            }
          }
          tmem_st_32x32b_x32(taddr + c * 32, r);
        }
        tmem_st_wait();
      }

      // ---- routing: which rank keeps this lane's row / this tile --------------
      int owner = p.rank;
      bool tile_reduces = false;            // uniform over the CTA
      bool tile_publishes = false;          // uniform over the CTA
      int o_lo = 0, o_hi = 0;
      // a CTA tile's later blocks can fall past the last row block
      const bool tile_has_rows = m_tile * BM < p.M;
      if (multi && tile_has_rows) {
        if (p.op == OP_RS && p.nvls) {
          // through the switch: every partial (own included) stays in this rank's own plane; the
          // communication warps of the rank that keeps the rows read the sum, no epilogue waits
          owner = min((m_tile * BM) / p.m_per_rank, p.R - 1);
          o_lo = o_hi = owner;
          tile_reduces = false;
          tile_publishes = true;
        } else if (p.op == OP_RS) {
          owner = min(row / p.m_per_rank, p.R - 1);
          o_lo = (m_tile * BM) / p.m_per_rank;
          o_hi = min((min(m_tile * BM + BM, p.M) - 1) / p.m_per_rank, p.R - 1);
          tile_reduces = (o_lo <= p.rank && p.rank <= o_hi);
          tile_publishes = !(o_lo == p.rank && o_hi == p.rank);
        } else if (p.op == OP_AR2) {
          // every partial (own included) goes to the owner's slot; the owner's communication
          // warps reduce and broadcast once all R partials are there, so no epilogue waits
          owner = t.owner_key % p.R;
          tile_reduces = false;
          tile_publishes = true;
        } else if (p.op == OP_AR1) {
          tile_reduces = true;
          tile_publishes = true;
        }
      }
      if (p.publish_only) tile_reduces = false;     // decomposition mode: publish and ticket, no reduce
      // Range check of the indices every later access of this block derives from (the plan was
      // checked on the host, the table-driven orders and the peers' shapes were not): a bad one
      // is recorded and nothing is accessed with it.
      if (multi && tile_has_rows && (tile_publishes || tile_reduces) &&
          (lin < 0 || lin >= tiles || owner < 0 || owner >= p.R)) {
        if (etid == 0) report_failure(env, ST_BAD_INDEX, SITE_INDEX_CHECK, static_cast<uint32_t>(tiles),
                                      static_cast<uint32_t>(lin), static_cast<uint32_t>(m_tile));
        alive = false;
        break;
      }
      // the accumulator is needed after the publish phase only where this rank adds the
      // peers' partials to it (its own rows of a reduce-scatter tile)
      const bool acc_needed_later = tile_reduces && p.op == OP_RS;

      // ---- phase 1: publish 16-bit partials into other ranks' slots --------------
      // Always before any wait: two owners of one mixed tile would otherwise wait
      // for each other's partial.
      const uint64_t t_pub0 = (prof && etid == 0) ? globaltimer_ns() : 0;
      if (kStaging && tile_publishes) {
        const bool one_dest_tile = (p.op != OP_RS) || (o_lo == o_hi);
        if (one_dest_tile) {
          // The whole tile goes to one rank (or, one-shot, to all of them): stage 128 columns
          // at a time in TMA layout and let one thread ship them with 2-D tiled stores
          // (two 128 x 64 boxes per destination) -- few large copy-engine operations.
          const int dest = (p.op == OP_RS) ? o_lo : owner;      // uniform over the CTA
          // peer slots hold the owner's rows only; a plane read through the switch holds all rows
          const int row0 = (p.op == OP_RS && !p.nvls) ? m_tile * BM - dest * p.m_per_rank : m_tile * BM;
          for (int half = 0; half < BN / kStageCols; ++half) {
            const int col0 = t.n_tile * BN + half * kStageCols;
            if (col0 >= p.N) break;
            if (lane == 0) tma_store_wait_read<0>();   // earlier stores have read the staging
            named_bar_sync(2, kEpiThreads);
#pragma unroll 1
            for (int c = 0; c < kStageCols / 32; ++c) {
              uint32_t r[32];
              tmem_ld_32x32b_x32(taddr + half * kStageCols + c * 32, r);
              tmem_ld_wait();
              float acc[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) acc[j] = __uint_as_float(r[j]);
              stage_row32_swizzled<kBf16>(staging, r_in_tile, c, acc);
            }
            fence_proxy_async_smem();
            named_bar_sync(2, kEpiThreads);
            if (etid == 0) {
              if (p.op == OP_AR1) {
                for (int d = 0; d < p.R; ++d) {
                  tma_store_2d(&p.tma_slot[d], staging, col0, row0);
                  tma_store_2d(&p.tma_slot[d], staging + kBoxBytes, col0 + 64, row0);
                }
              } else {
                tma_store_2d(&p.tma_slot[dest], staging, col0, row0);
                tma_store_2d(&p.tma_slot[dest], staging + kBoxBytes, col0 + 64, row0);
              }
              tma_store_commit();
            }
          }
          // the partial is in shared memory (or on its way): the MMAs of the next tile may
          // overwrite the accumulator while the stores complete and the ticket goes out
          if (!acc_needed_later) release_acc();
          if (prof && etid == 0) prof[PROF_TL_STAGED] = globaltimer_ns() - t_kernel0;
          if (etid == 0) tma_store_wait_all<0>();      // every byte has been written
          if (prof && etid == 0) prof[PROF_TL_STORED] = globaltimer_ns() - t_kernel0;
        } else {
          // Each thread owns one accumulator row: it converts 128 columns into its staging
          // row, then ships the 256 contiguous bytes to every destination with one bulk
          // copy each (large NVLink writes instead of scattered 16-byte stores).
          uint8_t* my_stage = staging + r_in_tile * kStagePitch;
          for (int half = 0; half < BN / kStageCols; ++half) {
            const int col0 = t.n_tile * BN + half * kStageCols;
            tma_store_wait_read<0>();          // my previous copies have read this row
#pragma unroll 1
            for (int c = 0; c < kStageCols / 32; ++c) {
              uint32_t r[32];
              tmem_ld_32x32b_x32(taddr + half * kStageCols + c * 32, r);
              tmem_ld_wait();
              uint4* d4 = reinterpret_cast<uint4*>(my_stage + c * 64);
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 o;
                o.x = pack2<kBf16>(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
                o.y = pack2<kBf16>(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
                o.z = pack2<kBf16>(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
                o.w = pack2<kBf16>(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
                d4[v] = o;
              }
            }
            fence_proxy_async_smem();          // generic smem writes -> visible to the bulk copy
            if (row_ok && col0 < p.N) {
              if (p.op == OP_AR1) {
                const int64_t off = static_cast<int64_t>(row) * p.N + col0;
                for (int d = 0; d < p.R; ++d)
                  bulk_store_1d(reinterpret_cast<uint8_t*>(p.peer_slots[d]) +
                                    (static_cast<int64_t>(p.rank) * p.slot_stride + off) * 2,
                                my_stage, kStageRowBytes);
              } else if (owner != p.rank || p.op == OP_AR2) {
                const int64_t off = (p.op == OP_RS)
                    ? static_cast<int64_t>(row - owner * p.m_per_rank) * p.N + col0
                    : static_cast<int64_t>(row) * p.N + col0;
                bulk_store_1d(reinterpret_cast<uint8_t*>(p.peer_slots[owner]) +
                                  (static_cast<int64_t>(p.rank) * p.slot_stride + off) * 2,
                              my_stage, kStageRowBytes);
              }
            }
            tma_store_commit();
          }
          if (!acc_needed_later) release_acc();
          tma_store_wait_all<0>();             // every byte has been written
        }
        // Every thread has seen its own bulk stores complete. The barrier orders them before the
        // ticket stores below, whose release (one system fence per storing warp, cumulative over
        // what the barrier ordered) publishes them: a fence in all 128 threads here cost 10-20 us.
        named_bar_sync(2, kEpiThreads);
        if (p.op == OP_RS) {
          const int o = o_lo + etid;
          if (o <= o_hi && (o != p.rank || p.nvls))
            st_release_sys(p.peer_tile_flags[o] + p.rank * tiles + lin, p.round);
        } else if (p.op == OP_AR1) {
          if (etid < p.R && etid != p.rank)
            st_release_sys(p.peer_tile_flags[etid] + p.rank * tiles + lin, p.round);
        } else if (etid == 0) {
          st_release_sys(p.peer_tile_flags[owner] + p.rank * tiles + lin, p.round);
        }
        if (prof && etid == 0) prof[PROF_TL_FLAGGED] = globaltimer_ns() - t_kernel0;
      }

      const uint64_t t_pub1 = (prof && etid == 0) ? globaltimer_ns() : 0;
      // ---- phase 2: wait for the other sources' partials of this tile -------------
      if (tile_reduces) {
        bool ok = true;
        if (etid == 0) {
          for (int s = 0; ok && s < p.R; ++s) {
            if (s == p.rank) continue;
            ok = wait_flag_ge(p.peer_tile_flags[p.rank] + s * tiles + lin, p.round, env,
                              p.op == OP_RS ? SITE_RS_TILE : SITE_AR_TILE, (s << 24) | lin);
          }
        }
        // the barriers inside the vote also order the slot reads after the acquire
        if (!epi_vote(s_flags, ok)) { alive = false; break; }
      }

      if (prof && etid == 0) {
        acc_pub += t_pub1 - t_pub0;
        acc_tick += globaltimer_ns() - t_pub1;
      }
      // ---- phase 3: final values of the rows / tile this rank keeps ---------------
      const bool finalizes =
          tile_has_rows && (!multi || p.op == OP_PLAIN || p.op == OP_AG || tile_reduces);
      if (finalizes) {
        // registers only inside the column loop: its inline-asm statements clobber memory, so
        // fields read through `p` there would be re-loaded for every 32-column chunk
        const int op = p.op;
        const bool swiglu = p.epi == EPI_SWIGLU;
        const int n_cols = p.N;
        uint8_t* const c_base = reinterpret_cast<uint8_t*>(p.c);
        const bool local_tile = !multi || op == OP_PLAIN || op == OP_AG;
        if (local_tile && staging_free && p.c_tma) {
          // Local result: every epilogue warp converts its 32 rows, 64 columns at a time, into
          // one of its two swizzled 32 x 64 boxes and ships the box with a 2-D tiled store of its
          // own (rows and columns past the end of c are clipped by the copy engine). The four
          // warps never meet at a barrier here, and the accumulator is free as soon as its last
          // columns are in shared memory; nobody waits for the stores.
          const int out_col0 = swiglu ? t.n_tile * (BN / 2) : t.n_tile * BN;
          constexpr int kWarpBox = 32 * 128;
          uint8_t* const wbox = staging + q * (2 * kWarpBox);
          const int out_row0 = m_tile * BM + q * 32;
          uint32_t rab[64];                  // accumulator columns in flight (plain store only)
#pragma unroll
          for (int j = 0; j < BN / 64; ++j) {
            if (swiglu && j >= BN / 128) break;
            const int ocol = out_col0 + j * 64;
            if (ocol >= n_cols) break;
            uint8_t* box = wbox + (j & 1) * kWarpBox;
            uint32_t pk[32];                 // 64 columns of this lane's row, packed to 16 bit
            if (swiglu) {
              // gate in accumulator columns [0, BN/2), up in [BN/2, BN)
#pragma unroll
              for (int cc = 0; cc < 2; ++cc) {
                uint32_t g[32], u[32];
                tmem_ld_32x32b_x32(taddr + j * 64 + cc * 32, g);
                tmem_ld_32x32b_x32(taddr + BN / 2 + j * 64 + cc * 32, u);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 16; ++e)
                  pk[cc * 16 + e] = pack2<kBf16>(silu(__uint_as_float(g[2 * e])) * __uint_as_float(u[2 * e]),
                                                 silu(__uint_as_float(g[2 * e + 1])) * __uint_as_float(u[2 * e + 1]));
              }
            } else {
              // the loads of box j were issued while box j - 1 was being staged
              if (j == 0) tmem_ld_32x32b_x64(taddr, rab);
              tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                pk[e] = pack2<kBf16>(__uint_as_float(rab[2 * e]), __uint_as_float(rab[2 * e + 1]));
                pk[16 + e] = pack2<kBf16>(__uint_as_float(rab[32 + 2 * e]), __uint_as_float(rab[32 + 2 * e + 1]));
              }
              if (j + 1 < BN / 64 && out_col0 + (j + 1) * 64 < n_cols)
                tmem_ld_32x32b_x64(taddr + (j + 1) * 64, rab);
            }
            // the store that last read this box was issued two groups ago (any group for j = 0)
            if (lane == 0) {
              if (j == 0) tma_store_wait_read<0>();
              else tma_store_wait_read<1>();
            }
            __syncwarp();
#pragma unroll
            for (int v = 0; v < 8; ++v)
              *reinterpret_cast<uint4*>(box + lane * 128 + ((v ^ (lane & 7)) * 16)) =
                  make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&p.tma_c32, box, ocol, out_row0);
              tma_store_commit();
            }
          }
        } else {
        for (int c = 0; c < BN / 32; ++c) {
          if (swiglu && c >= BN / 64) break;
          const int ocol = swiglu ? t.n_tile * (BN / 2) + c * 32 : t.n_tile * BN + c * 32;
          float acc[32];
          if (multi && op == OP_AR1) {
            // all R contributions (own included) are summed from their 16-bit form
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] = 0.f;
          } else if (swiglu) {
            // gate in accumulator columns [0, BN/2), up in [BN/2, BN)
            uint32_t g[32], u[32];
            tmem_ld_32x32b_x32(taddr + c * 32, g);
            tmem_ld_32x32b_x32(taddr + BN / 2 + c * 32, u);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j)
              acc[j] = silu(__uint_as_float(g[j])) * __uint_as_float(u[j]);
          } else {
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] = __uint_as_float(r[j]);
          }
          const bool active = row_ok && ocol < n_cols;
          if (active) {
            if (local_tile) {
              // (N is a multiple of 8, not necessarily of 32: the last chunk of a row can be short)
              store_row32<kBf16>(c_base + (static_cast<int64_t>(row) * ldc + ocol) * 2, acc, n_cols - ocol);
            } else if (op == OP_RS) {
              if (owner == p.rank) {
                const int lrow = row - owner * p.m_per_rank;
                // fixed source order keeps the sum deterministic
                add_rows32_from_sources<kBf16>(
                    acc, reinterpret_cast<const uint8_t*>(p.peer_slots[p.rank]) +
                             (static_cast<int64_t>(lrow) * p.N + ocol) * 2,
                    p.slot_stride * 2, p.R, p.rank);
                store_row32<kBf16>(reinterpret_cast<uint8_t*>(p.c) +
                                       (static_cast<int64_t>(lrow) * ldc + ocol) * 2,
                                   acc);
              }
            } else if (op == OP_AR1) {
              const int64_t off = static_cast<int64_t>(row) * n_cols + ocol;
              add_rows32_from_sources<kBf16>(
                  acc, reinterpret_cast<const uint8_t*>(p.peer_slots[p.rank]) + off * 2,
                  p.slot_stride * 2, p.R, -1);
              store_row32<kBf16>(reinterpret_cast<uint8_t*>(p.c) +
                                     (static_cast<int64_t>(row) * ldc + ocol) * 2,
                                 acc);
            }
          }
        }
        }
      }

      if (!released) release_acc();
      if (prof && etid == 0) {
        acc_busy += globaltimer_ns() - t_epi0;
        ++n_tiles_done;
      }
      }   // 128-row blocks of the CTA tile
      ++it;
    }
    // staged stores must have read shared memory before the CTA goes away
    if (kStaging && lane == 0) tma_store_wait_all<0>();
    if (prof && etid == 0) {
      prof[PROF_EPI_BUSY] = acc_busy;
      prof[PROF_EPI_PUBLISH] = acc_pub;
      prof[PROF_EPI_TICKET_WAIT] = acc_tick;
      prof[PROF_EPI_TILES] = n_tiles_done;
      prof[PROF_SK_WAIT] = acc_sk;
      prof[PROF_EPI_DONE_AT] = globaltimer_ns() - t_kernel0;
    }
  }
  // ==========================================================================
  // warps 6-9: communication
  // ==========================================================================
  else {
    const int ctid = threadIdx.x - kCommWarp0 * 32;
    if (kStaging && p.op == OP_AG && p.R > 1 && !p.skip_comm) {
      // Push this rank's shard to every peer, nearest-next rank first, so that at any
      // moment each rank receives from exactly one sender. One work item is one `part`
      // of one chunk for one destination. A single thread drives the copy engine of
      // the SM: 16 KB pieces are bulk-loaded into a ring of kPushSlots slots and bulk-stored
      // to the peer, so the push costs no load/store-unit bandwidth and NVLink sees large
      // writes. The ring is the operand ring of the GEMM: a pushing CTA computes nothing until
      // its part of the push is done (its producer warp waits for s_flags[2]), which gives the
      // copy engine a dozen pieces in flight instead of two and keeps the push from competing
      // with the CTA's own operand loads.
      if (p.ag_mc) {
        // ---- multicast push: one store through the switch reaches every rank's workspace, so this
        // rank sends its shard ONCE (not once per peer). The communication warps of the first
        // push_grid CTAs do it (registers only, no shared memory); those CTAs join the GEMM when
        // their part is out, like the CTAs of the bulk-copy push, but there are fewer bytes to
        // wait for. Chunk-major, each sending CTA a slice of every chunk, so that the first rows
        // are complete everywhere first; the last CTA to finish its slice of a chunk raises that
        // chunk's ticket on all peers.
        constexpr int kU = 8;                                        // 16-byte pieces in flight per thread
        const int64_t chunk_pieces = static_cast<int64_t>(p.chunk_rows) * p.K / 8;
        const int64_t per = (chunk_pieces + push_grid - 1) / push_grid;
        const int64_t lo_in = min(chunk_pieces, per * static_cast<int64_t>(blockIdx.x));
        const int64_t hi_in = min(chunk_pieces, lo_in + per);
        const uint8_t* const src = reinterpret_cast<const uint8_t*>(p.a_local);
        uint8_t* const dst = reinterpret_cast<uint8_t*>(p.mc_part) +
                             static_cast<int64_t>(p.rank) * p.m_per_rank * p.K * 2;
        for (int ck = 0; pushes && ck < p.n_chunks; ++ck) {
          const int64_t lo = ck * chunk_pieces + lo_in, hi = ck * chunk_pieces + hi_in;
          for (int64_t base = lo + ctid; base < hi; base += static_cast<int64_t>(kCommThreads) * kU) {
            uint4 v[kU];
#pragma unroll
            for (int u = 0; u < kU; ++u) {        // (index clamped: no branch between the loads)
              const int64_t i = min(base + static_cast<int64_t>(u) * kCommThreads, hi - 1);
              v[u] = ld_global_nc_v4(src + i * 16);
            }
#pragma unroll
            for (int u = 0; u < kU; ++u) {
              const int64_t i = base + static_cast<int64_t>(u) * kCommThreads;
              if (i < hi) multimem_st_v4(dst + i * 16, v[u]);
            }
          }
          // the counter add below releases what this barrier ordered (all 128 threads' stores)
          named_bar_sync(1, kCommThreads);
          if (ctid == 0) {
            uint32_t* cnt = p.ag_counters + ck;
            if (atom_add_acq_rel_gpu(cnt, 1u) + 1u == static_cast<uint32_t>(push_grid)) {
              atomicExch(cnt, 0u);
              for (int d = 0; d < p.R; ++d)
                if (d != p.rank) st_release_sys(p.peer_ag_flags[d] + p.rank * p.ag_flag_stride + ck, p.round);
            }
          }
        }
        if (pushes) {
          named_bar_sync(1, kCommThreads);
          if (ctid == 0) {
            __threadfence_block();
            s_flags[2] = 1;               // this CTA's producer may start
          }
        }
      } else if (ctid == 0) {
        constexpr uint32_t kPiece = 16384;
        constexpr int kLag = kPushSlots / 2;     // stores that may still be reading their slot
        static_assert(kPushSlots * kPiece <= TS::kStages * TS::kStageBytes, "push ring exceeds the operand ring");
        const int64_t chunk_bytes = static_cast<int64_t>(p.chunk_rows) * p.K * 2;
        const int64_t part_bytes = chunk_bytes / p.push_parts;   // host guarantees % 16 == 0
        const int items_per_dest = p.n_chunks * p.push_parts;
        const int pieces = static_cast<int>((part_bytes + kPiece - 1) / kPiece);
        uint32_t par_mask = 0u;                  // phase parity of every slot's barrier
        bool ok = true;
        auto piece_bytes = [&](int i) -> uint32_t {
          const int64_t left = part_bytes - static_cast<int64_t>(i) * kPiece;
          return static_cast<uint32_t>(left < kPiece ? left : kPiece);
        };
        // one part (part_bytes) from src to dst through the ring; returns once every byte is written
        auto copy_part = [&](const uint8_t* src, uint8_t* dst) {
          auto load_piece = [&](int i) {
            const int sl = i % kPushSlots;
            mbar_arrive_expect_tx(&push_bar[sl], piece_bytes(i));
            bulk_load_1d(ring + sl * kPiece, src + static_cast<int64_t>(i) * kPiece, piece_bytes(i), &push_bar[sl]);
          };
          // all stores of the previous part were drained: every slot is free
          for (int i = 0; i < kPushSlots && i < pieces; ++i) load_piece(i);
          for (int i = 0; ok && i < pieces; ++i) {
            const int sl = i % kPushSlots;
            ok = wait_mbar(&push_bar[sl], (par_mask >> sl) & 1u, env, SITE_PIPE_FULL, 100 + sl);
            par_mask ^= 1u << sl;
            if (!ok) break;
            bulk_store_1d(dst + static_cast<int64_t>(i) * kPiece, ring + sl * kPiece, piece_bytes(i));
            tma_store_commit();
            // the store of piece i - kLag has read its slot once at most kLag newer stores are
            // still reading theirs: refill that slot with the piece one ring turn later
            const int j = i - kLag;
            if (j >= 0 && j + kPushSlots < pieces) {
              tma_store_wait_read<kLag>();
              load_piece(j + kPushSlots);
            }
          }
          tma_store_wait_all<0>();             // every byte of the part has been written
        };
        // counts a finished part of chunk (row, ck) in; true for the thread that completes the chunk
        auto chunk_done = [&](int row, int ck) -> bool {
          fence_acq_rel_sys();
          uint32_t* cnt = p.ag_counters + row * p.n_chunks + ck;
          const uint32_t old = atomicAdd(cnt, 1u);
          if (old + 1u != static_cast<uint32_t>(p.push_parts)) return false;
          atomicExch(cnt, 0u);
          fence_acq_rel_sys();
          return true;
        };
        const int64_t my_slot_off = static_cast<int64_t>(p.rank) * p.m_per_rank * p.K * 2;
        if (!p.ag_pull) {
          // ---- push: my shard into every peer's workspace, the peer's ticket when a chunk is in ----
          const int items = (p.R - 1) * items_per_dest;
          for (int item = blockIdx.x; ok && pushes && item < items; item += push_grid) {
            const int di = item / items_per_dest;
            const int rem = item - di * items_per_dest;
            const int ck = rem / p.push_parts;
            const int part = rem - ck * p.push_parts;
            const int dest = (p.rank + 1 + di) % p.R;
            const int64_t off = ck * chunk_bytes + part * part_bytes;
            copy_part(reinterpret_cast<const uint8_t*>(p.a_local) + off,
                      reinterpret_cast<uint8_t*>(p.peer_ws[dest]) + my_slot_off + off);
            if (!ok) break;                    // (a wait ran out: its status is recorded)
            if (chunk_done(dest, ck))
              st_release_sys(p.peer_ag_flags[dest] + p.rank * p.ag_flag_stride + ck, p.round);
          }
        } else {
          // ---- pull (the reference's tile-ready transport, gemm_ag_tr.py:407-449): every rank
          // stages its shard in its own workspace and tells the peers chunk by chunk ("arrive");
          // every rank then copies the peers' chunks out of their workspaces into its own and
          // raises its own ready ticket, the one the consumer waits for.
          for (int item = blockIdx.x; ok && pushes && item < items_per_dest; item += push_grid) {
            const int ck = item / p.push_parts;
            const int part = item - ck * p.push_parts;
            const int64_t off = ck * chunk_bytes + part * part_bytes;
            copy_part(reinterpret_cast<const uint8_t*>(p.a_local) + off,
                      reinterpret_cast<uint8_t*>(p.peer_ws[p.rank]) + my_slot_off + off);
            if (!ok) break;
            if (chunk_done(p.R, ck))           // (row R of the counters: the staging of my own shard)
              for (int d = 0; d < p.R; ++d)
                if (d != p.rank) st_release_sys(p.peer_ag_arrive[d] + p.rank * p.ag_flag_stride + ck, p.round);
          }
          const int items = (p.R - 1) * items_per_dest;
          for (int item = blockIdx.x; ok && pushes && item < items; item += push_grid) {
            const int di = item / items_per_dest;
            const int rem = item - di * items_per_dest;
            const int ck = rem / p.push_parts;
            const int part = rem - ck * p.push_parts;
            const int src = (p.rank + p.R - 1 - di) % p.R;      // nearest previous rank first: the consumer's order
            ok = wait_flag_ge(p.peer_ag_arrive[p.rank] + src * p.ag_flag_stride + ck, p.round, env, SITE_AG_ARRIVE,
                              (src << 16) | ck);
            if (!ok) break;
            const int64_t off = static_cast<int64_t>(src) * p.m_per_rank * p.K * 2 + ck * chunk_bytes + part * part_bytes;
            copy_part(reinterpret_cast<const uint8_t*>(p.peer_ws[src]) + off,
                      reinterpret_cast<uint8_t*>(p.peer_ws[p.rank]) + off);
            if (!ok) break;
            if (chunk_done(src, ck))
              st_release_sys(p.peer_ag_flags[p.rank] + src * p.ag_flag_stride + ck, p.round);
          }
        }
        // every copy of this thread has completed (or the transfer gave up): the operand ring and
        // the staging area now belong to the GEMM roles of this CTA
        __threadfence_block();
        s_flags[2] = 1;
      }
    } else if (p.op == OP_RS && p.nvls && p.R > 1) {
      // Reduce-scatter through the switch: the 128-row blocks of this rank's own rows, in the
      // order all ranks compute them, spread over the CTAs. Wait for the R partial tickets of a
      // block, read the SUM of the R ranks' partials with multimem.ld_reduce (added inside the
      // switch, fp32 accumulation) and store it into c.
      const int per_seg = p.seg_m_tiles * p.n_tiles;
      bool ok = true;
      int owned_seq = 0;
      const bool cprof = prof && ctid == 0;
      uint64_t acc_aw = 0, acc_ak = 0;
      uint8_t* const mc_in = reinterpret_cast<uint8_t*>(p.mc_part);
      // Reduce budget (the steady / tail CTA budget of the reference's windowed reduce-scatter,
      // gemm_rs_v5.py:489-501): the first blocks are reduced by `reduce_ctas` CTAs only, the last
      // `reduce_tail` blocks by every CTA of the grid, when nothing is left to compute.
      const int all_ctas = static_cast<int>(gridDim.x);
      const int steady = (p.reduce_ctas > 0 && p.reduce_ctas < all_ctas) ? p.reduce_ctas : all_ctas;
      const int n_owned = per_seg * p.sub_tiles;
      const int tail0 = n_owned - ((steady < all_ctas) ? max(p.reduce_tail, 0) : 0);
      for (int u = 0; ok && u < per_seg; ++u) {
        int um, nt;
        raster_grouped(u, p.seg_m_tiles, p.n_tiles, p.raster_g, um, nt);
        for (int subt = 0; ok && subt < p.sub_tiles; ++subt, ++owned_seq) {
          const int team = owned_seq < tail0 ? steady : all_ctas;
          if (owned_seq % team != static_cast<int>(blockIdx.x)) continue;
          const int mt = (p.rank * p.seg_m_tiles + um) * p.sub_tiles + subt;
          if (mt * BM >= p.M) continue;
          const int lin = mt * p.n_tiles + nt;
          const uint64_t ta0 = cprof ? globaltimer_ns() : 0;
          if (ctid == 0) s_flags[1] = 1;
          named_bar_sync(1, kCommThreads);
          if (ctid < p.R &&
              !wait_flag_ge(p.peer_tile_flags[p.rank] + ctid * p.ticket_stride + lin, p.round, env, SITE_RS_TILE,
                            (ctid << 24) | lin))
            s_flags[1] = 0;
          named_bar_sync(1, kCommThreads);     // also orders the reads below after the acquires
          ok = s_flags[1] != 0;
          named_bar_sync(1, kCommThreads);
          if (!ok) break;
          const uint64_t ta1 = cprof ? globaltimer_ns() : 0;
          const int rows = min(BM, p.M - mt * BM);
          const int cols = min(BN, p.N - nt * BN);
          const int vpr = cols >> 3;
          const int total = rows * vpr;
          const int lrow0 = mt * BM - p.rank * p.m_per_rank;
          constexpr int kU = 16;
          for (int i0 = ctid; i0 < total; i0 += kU * kCommThreads) {
            uint4 val[kU];
            // all loads of the batch are issued before the first store needs its value; pieces
            // past the end of the block re-read its last piece (no branch between the loads)
#pragma unroll
            for (int u2 = 0; u2 < kU; ++u2) {
              const int idx = min(i0 + u2 * kCommThreads, total - 1);
              const int r = idx / vpr;
              const int v = idx - r * vpr;
              const int64_t off = static_cast<int64_t>(mt * BM + r) * p.N + nt * BN + v * 8;
              val[u2] = multimem_ld_reduce_add_v4<kBf16>(mc_in + off * 2);
            }
#pragma unroll
            for (int u2 = 0; u2 < kU; ++u2) {
              const int idx = i0 + u2 * kCommThreads;
              if (idx >= total) break;
              const int r = idx / vpr;
              const int v = idx - r * vpr;
              st_global_v4(reinterpret_cast<uint8_t*>(p.c) +
                               (static_cast<int64_t>(lrow0 + r) * p.ldc + nt * BN + v * 8) * 2,
                           val[u2]);
            }
          }
          if (cprof) {
            acc_aw += ta1 - ta0;
            acc_ak += globaltimer_ns() - ta1;
          }
        }
      }
      if (cprof) {
        prof[PROF_AR_A_WAIT] = acc_aw;
        prof[PROF_AR_A_WORK] = acc_ak;
        prof[PROF_AR_A_DONE_AT] = globaltimer_ns() - t_kernel0;
      }
    } else if (p.op == OP_AR2 && p.R > 1 && !p.publish_only) {
      const int tickets = p.unit_m * p.sub_tiles * p.n_tiles;
      const int units = p.unit_m * p.n_tiles;
      bool ok = true;
      // ---- phase A: finish the tiles this rank owns (unit % R == rank), spread over all CTAs --
      // wait for the R partials of a tile, sum them in fp32 in source order, write the result
      // into every rank's result buffer with coalesced 16-byte stores, raise the result tickets
      int owned_seq = 0;
      const bool cprof = prof && ctid == 0;
      if (cprof) prof[PROF_TL_COMM_START] = globaltimer_ns() - t_kernel0;
      uint64_t acc_aw = 0, acc_ak = 0, acc_bw = 0, acc_bc = 0;
      for (int unit = p.rank; ok && unit < units; unit += p.R) {
        for (int subt = 0; ok && subt < p.sub_tiles; ++subt, ++owned_seq) {
          if (owned_seq % static_cast<int>(gridDim.x) != static_cast<int>(blockIdx.x)) continue;
          const int lin = unit * p.sub_tiles + subt;
          int um, nt;
          raster_grouped(unit, p.unit_m, p.n_tiles, p.raster_g, um, nt);
          const int mt = um * p.sub_tiles + subt;
          if (mt * BM >= p.M) continue;
          const uint64_t ta0 = cprof ? globaltimer_ns() : 0;
          if (ctid == 0) s_flags[1] = 1;
          named_bar_sync(1, kCommThreads);
          if (ctid < p.R &&
              !wait_flag_ge(p.peer_tile_flags[p.rank] + ctid * p.ticket_stride + lin, p.round, env, SITE_AR_TILE,
                            (ctid << 24) | lin))
            s_flags[1] = 0;
          named_bar_sync(1, kCommThreads);     // also orders the slot reads after the acquires
          ok = s_flags[1] != 0;
          named_bar_sync(1, kCommThreads);
          if (!ok) break;
          const uint64_t ta1 = cprof ? globaltimer_ns() : 0;
          if (cprof) prof[PROF_TL_OWN_SEEN] = ta1 - t_kernel0;
          const int rows = min(BM, p.M - mt * BM);
          const int cols = min(BN, p.N - nt * BN);
          const int vpr = cols >> 3;
          const int total = rows * vpr;
          if (p.nvls) {
            // the switch adds the R copies of a 16-byte piece on the way here and replicates
            // the result on the way back: one load and one store per piece, whatever R is
            constexpr int kU = 16;
            uint8_t* mc_in = reinterpret_cast<uint8_t*>(p.mc_part);
            uint8_t* mc_out = reinterpret_cast<uint8_t*>(p.mc_res);
            for (int i0 = ctid; i0 < total; i0 += kU * kCommThreads) {
              uint4 val[kU];
              // all loads of the batch are issued before the first store needs its value; pieces
              // past the end of the tile re-read its last piece (no branch between the loads)
#pragma unroll
              for (int u = 0; u < kU; ++u) {
                const int idx = min(i0 + u * kCommThreads, total - 1);
                const int r = idx / vpr;
                const int v = idx - r * vpr;
                const int64_t off = static_cast<int64_t>(mt * BM + r) * p.N + nt * BN + v * 8;
                val[u] = multimem_ld_reduce_add_v4<kBf16>(mc_in + off * 2);
              }
#pragma unroll
              for (int u = 0; u < kU; ++u) {
                const int idx = i0 + u * kCommThreads;
                if (idx >= total) break;
                const int r = idx / vpr;
                const int v = idx - r * vpr;
                const int64_t row = mt * BM + r, col = nt * BN + v * 8;
                multimem_st_v4(mc_out + (row * p.N + col) * 2, val[u]);
                if (!p.res_is_c)
                  st_global_v4(reinterpret_cast<uint8_t*>(p.c) + (row * p.ldc + col) * 2, val[u]);
              }
              if (cprof && i0 == ctid) prof[PROF_TL_OWN_IT0] = globaltimer_ns() - t_kernel0;
            }
          } else {
          const uint8_t* slots = reinterpret_cast<const uint8_t*>(p.peer_slots[p.rank]);
          const int64_t sstride = p.slot_stride * 2;
          for (int i0 = ctid; i0 < total; i0 += 2 * kCommThreads) {
            float acc[2][8];
            int64_t off[2];
            bool on[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int idx = i0 + u * kCommThreads;
              on[u] = idx < total;
              const int r = on[u] ? idx / vpr : 0;
              const int v = on[u] ? idx - r * vpr : 0;
              off[u] = static_cast<int64_t>(mt * BM + r) * p.N + nt * BN + v * 8;
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
            }
            for (int s0 = 0; s0 < p.R; s0 += 4) {
              uint4 val[2][4];
#pragma unroll
              for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int k = 0; k < 4; ++k)
                  val[u][k] = (on[u] && s0 + k < p.R)
                                  ? ld_global_cg_v4(slots + (s0 + k) * sstride + off[u] * 2)
                                  : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
              for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  const uint32_t w[4] = {val[u][k].x, val[u][k].y, val[u][k].z, val[u][k].w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float2 f = unpack2<kBf16>(w[j]);
                    acc[u][2 * j] += f.x;
                    acc[u][2 * j + 1] += f.y;
                  }
                }
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              if (!on[u]) continue;
              uint4 o;
              o.x = pack2<kBf16>(acc[u][0], acc[u][1]);
              o.y = pack2<kBf16>(acc[u][2], acc[u][3]);
              o.z = pack2<kBf16>(acc[u][4], acc[u][5]);
              o.w = pack2<kBf16>(acc[u][6], acc[u][7]);
              for (int d = 0; d < p.R; ++d) {
                if (d == p.rank && !p.res_is_c) continue;
                st_global_v4(reinterpret_cast<uint8_t*>(p.peer_res[d]) + off[u] * 2, o);
              }
              if (!p.res_is_c) {
                const int64_t row = off[u] / p.N, col = off[u] - row * p.N;
                st_global_v4(reinterpret_cast<uint8_t*>(p.c) + (row * p.ldc + col) * 2, o);
              }
            }
            if (cprof && i0 == ctid) prof[PROF_TL_OWN_IT0] = globaltimer_ns() - t_kernel0;
          }
          }
          if (cprof) prof[PROF_TL_OWN_LOADED] = globaltimer_ns() - t_kernel0;
          // the releases below (one warp) are cumulative over the stores this barrier orders
          named_bar_sync(1, kCommThreads);
          if (cprof) prof[PROF_TL_OWN_FENCED] = globaltimer_ns() - t_kernel0;
          // the owner's row of the plane: one writer per word, whatever the shapes of earlier calls
          if (ctid < p.R && ctid != p.rank)
            st_release_sys(p.peer_res_flags[ctid] + p.rank * p.ticket_stride + lin, p.round);
          if (cprof) {
            prof[PROF_TL_OWN_FLAGGED] = globaltimer_ns() - t_kernel0;
            acc_aw += ta1 - ta0;
            acc_ak += globaltimer_ns() - ta1;
          }
        }
      }
      if (cprof) {
        prof[PROF_AR_A_WAIT] = acc_aw;
        prof[PROF_AR_A_WORK] = acc_ak;
        prof[PROF_AR_A_DONE_AT] = globaltimer_ns() - t_kernel0;
      }
      // ---- phase B: collect the tiles the other ranks finished ------------------------------
      for (int lin = blockIdx.x; ok && lin < tickets; lin += gridDim.x) {
        const int unit = lin / p.sub_tiles;
        if (unit % p.R == p.rank) continue;
        int um, nt;
        raster_grouped(unit, p.unit_m, p.n_tiles, p.raster_g, um, nt);
        const int mt = um * p.sub_tiles + (lin - unit * p.sub_tiles);
        if (mt * BM >= p.M) continue;         // nothing is ever published for an empty row block
        const uint64_t tb0 = cprof ? globaltimer_ns() : 0;
        if (ctid == 0)
          ok = wait_flag_ge(p.peer_res_flags[p.rank] + (unit % p.R) * p.ticket_stride + lin, p.round, env,
                            SITE_AR_RESULT, lin);
        // all comm threads learn the outcome; also orders their loads after the acquire
        if (ctid == 0) s_flags[1] = ok ? 1 : 0;
        named_bar_sync(1, kCommThreads);
        ok = s_flags[1] != 0;
        named_bar_sync(1, kCommThreads);
        const uint64_t tb1 = cprof ? globaltimer_ns() : 0;
        if (cprof) {
          acc_bw += tb1 - tb0;
          prof[PROF_TL_COL_SEEN] = tb1 - t_kernel0;
        }
        if (!ok || p.res_is_c) continue;
        const int rows = min(BM, p.M - mt * BM);
        const int cols = min(BN, p.N - nt * BN);
        const int v_per_row = cols >> 3;
        const int total = rows * v_per_row;
        for (int i0 = ctid; i0 < total; i0 += 8 * kCommThreads) {
          uint4 val[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int idx = i0 + u * kCommThreads;
            if (idx < total) {
              const int r = idx / v_per_row;
              const int v = idx - r * v_per_row;
              const int64_t off = static_cast<int64_t>(mt * BM + r) * p.N + nt * BN + v * 8;
              val[u] = ld_global_cg_v4(reinterpret_cast<const uint8_t*>(p.peer_res[p.rank]) + off * 2);
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int idx = i0 + u * kCommThreads;
            if (idx < total) {
              const int r = idx / v_per_row;
              const int v = idx - r * v_per_row;
              st_global_v4(reinterpret_cast<uint8_t*>(p.c) +
                               (static_cast<int64_t>(mt * BM + r) * p.ldc + nt * BN + v * 8) * 2,
                           val[u]);
            }
          }
        }
        if (cprof) acc_bc += globaltimer_ns() - tb1;
      }
      if (cprof) {
        prof[PROF_AR_B_WAIT] = acc_bw;
        prof[PROF_AR_B_COPY] = acc_bc;
      }
    }
  }


  if (prof && threadIdx.x == kCommWarp0 * 32)
    prof[PROF_PUSH_TOTAL] = globaltimer_ns() - (p.prof ? t_kernel0 : 0);
  // ==========================================================================
  // teardown
  // ==========================================================================
  // A pair leaves together: neither CTA may exit while the other can still signal its
  // barriers or issue MMAs that write its tensor memory.
  tc_fence_before_sync();
  if constexpr (kCtaM == 2) cluster_sync_all();
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    if constexpr (kCtaM == 2) tmem_dealloc_pair(tmem_base, TS::kTmemCols);
    else tmem_dealloc(tmem_base, TS::kTmemCols);
  }
  if (prof && threadIdx.x == 0) {
    const uint64_t t_end = globaltimer_ns();
    prof[PROF_KERNEL] = t_end - t_kernel0;
    prof[PROF_T_ENTRY] = t_entry;
    prof[PROF_T_SETUP] = t_kernel0;
    prof[PROF_T_END] = t_end;
  }
}

}  // namespace tdb
