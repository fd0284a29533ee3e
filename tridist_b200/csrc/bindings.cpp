// Python bindings (module `tridist_b200._C`): the native layer under tridist_b200/parallel and
// tridist_b200/ops, where the reference binds its host library through ctypes
// (pydushmem/host.py:64-301).
#include <c10/cuda/CUDAStream.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "ops/elementwise.h"
#include "ops/fused_gemm.h"
#include "ops/moe_a2a.h"
#include "ops/rd_exchange.h"
#include "common/status.h"
#include "runtime/symm_heap.h"
#include "runtime/vmm_heap.h"

namespace py = pybind11;
using namespace tdb;

static void* cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

template <typename T>
static T get(const py::dict& d, const char* k, T dflt) {
  if (!d.contains(k)) return dflt;
  return d[k].cast<T>();
}

static void fill_ptrs(const py::dict& d, const char* k, int64_t* out, int n) {
  if (!d.contains(k)) return;
  auto v = d[k].cast<std::vector<int64_t>>();
  for (int i = 0; i < n && i < static_cast<int>(v.size()); ++i) out[i] = v[i];
}

static void fill_ptrs2(const py::dict& d, const char* k, int64_t (*out)[8]) {
  if (!d.contains(k)) return;
  auto v = d[k].cast<std::vector<std::vector<int64_t>>>();
  for (int p = 0; p < 2 && p < static_cast<int>(v.size()); ++p)
    for (int i = 0; i < 8 && i < static_cast<int>(v[p].size()); ++i) out[p][i] = v[p][i];
}

static GemmPlanDesc gemm_desc_from(const py::dict& d) {
  GemmPlanDesc g;
  g.op = get<int>(d, "op", 0);
  g.epi = get<int>(d, "epi", 0);
  g.sched = get<int>(d, "sched", 0);
  g.bn = get<int>(d, "bn", 256);
  g.bf16 = get<bool>(d, "bf16", false);
  g.rank = get<int>(d, "rank", 0);
  g.R = get<int>(d, "R", 1);
  g.M = get<int>(d, "M", 0);
  g.N = get<int>(d, "N", 0);
  g.K = get<int>(d, "K", 0);
  g.a = get<int64_t>(d, "a", 0);
  g.a_rows = get<int64_t>(d, "a_rows", g.M);
  g.lda = get<int64_t>(d, "lda", g.K);
  g.b = get<int64_t>(d, "b", 0);
  g.b_rows = get<int64_t>(d, "b_rows", g.N);
  g.ldb = get<int64_t>(d, "ldb", g.K);
  g.c = get<int64_t>(d, "c", 0);
  g.ldc = get<int64_t>(d, "ldc", g.N);
  g.m_per_rank = get<int>(d, "m_per_rank", 0);
  if (d.contains("seg_order")) {
    auto v = d["seg_order"].cast<std::vector<int>>();
    for (size_t i = 0; i < v.size() && i < 8; ++i) g.seg_order[i] = v[i];
  }
  g.order_table = get<int64_t>(d, "order_table", 0);
  g.order_table_header = get<int>(d, "order_table_header", 0);
  g.check_residency = get<int>(d, "check_residency", 0);
  g.strided_interleave = get<int>(d, "strided_interleave", 0);
  g.seg_interleave = get<int>(d, "seg_interleave", 0);
  g.seg_bands = get<int>(d, "seg_bands", 0);
  g.seg_own_first = get<int>(d, "seg_own_first", 0);
  fill_ptrs(d, "peer_abort", g.peer_abort, 8);
  g.tile_list = get<int64_t>(d, "tile_list", 0);
  g.list_len = get<int>(d, "list_len", 0);
  g.swiglu_up_row0 = get<int>(d, "swiglu_up_row0", 0);
  g.max_ctas = get<int>(d, "max_ctas", 0);
  g.allow_pair = get<int>(d, "allow_pair", 1);
  g.allow_wide = get<int>(d, "allow_wide", 1);
  g.allow_splitk = get<int>(d, "allow_splitk", 1);
  g.raster_g = get<int>(d, "raster_g", 0);
  g.l2_ahead = get<int>(d, "l2_ahead", 0);
  fill_ptrs2(d, "peer_ws", g.peer_ws);
  fill_ptrs(d, "peer_ag_flags", g.peer_ag_flags, 8);
  fill_ptrs(d, "peer_ag_arrive", g.peer_ag_arrive, 8);
  g.ag_pull = get<int>(d, "ag_pull", 0);
  g.ag_counters = get<int64_t>(d, "ag_counters", 0);
  g.arrival_ns = get<int64_t>(d, "arrival_ns", 0);
  g.chunk_rows = get<int>(d, "chunk_rows", 0);
  g.n_chunks = get<int>(d, "n_chunks", 0);
  g.push_parts = get<int>(d, "push_parts", 0);
  g.skip_comm = get<int>(d, "skip_comm", 0);
  g.push_ctas = get<int>(d, "push_ctas", 0);
  g.push_skip_rounds = get<int>(d, "push_skip_rounds", 0);
  fill_ptrs2(d, "peer_slots", g.peer_slots);
  fill_ptrs(d, "peer_tile_flags", g.peer_tile_flags, 8);
  g.slot_stride = get<int64_t>(d, "slot_stride", 0);
  g.ticket_stride = get<int>(d, "ticket_stride", 0);
  g.ag_flag_stride = get<int>(d, "ag_flag_stride", 0);
  fill_ptrs2(d, "peer_res", g.peer_res);
  fill_ptrs(d, "peer_res_flags", g.peer_res_flags, 8);
  g.res_is_c = get<int>(d, "res_is_c", 0);
  g.nvls = get<int>(d, "nvls", 0);
  g.reduce_ctas = get<int>(d, "reduce_ctas", 0);
  g.reduce_tail = get<int>(d, "reduce_tail", 0);
  if (d.contains("mc_part")) {
    auto v = d["mc_part"].cast<std::vector<int64_t>>();
    for (size_t i = 0; i < v.size() && i < 2; ++i) g.mc_part[i] = v[i];
  }
  if (d.contains("mc_res")) {
    auto v = d["mc_res"].cast<std::vector<int64_t>>();
    for (size_t i = 0; i < v.size() && i < 2; ++i) g.mc_res[i] = v[i];
  }
  g.prof = get<int64_t>(d, "prof", 0);
  g.status_dev = get<int64_t>(d, "status_dev", 0);
  g.abort_word = get<int64_t>(d, "abort_word", 0);
  g.timeout_ns = get<uint64_t>(d, "timeout_ns", 2000000000ull);
  g.poll_ns = get<uint32_t>(d, "poll_ns", 0u);
  g.probe = get<int>(d, "probe", 0);
  return g;
}

static int64_t py_gemm_plan_create(const py::dict& d) { return gemm_plan_create(gemm_desc_from(d)); }

static std::vector<std::string> py_plan_check(const py::dict& d, const py::dict& ext, int sms) {
  PlanExtents e;
  e.c_bytes = get<int64_t>(ext, "c_bytes", 0);
  e.ws_bytes = get<int64_t>(ext, "ws_bytes", 0);
  e.slot_bytes = get<int64_t>(ext, "slot_bytes", 0);
  e.res_bytes = get<int64_t>(ext, "res_bytes", 0);
  e.ag_flag_words = get<int64_t>(ext, "ag_flag_words", 0);
  e.tile_flag_words = get<int64_t>(ext, "tile_flag_words", 0);
  e.res_flag_words = get<int64_t>(ext, "res_flag_words", 0);
  return plan_check(gemm_desc_from(d), e, sms);
}

static std::vector<std::vector<std::array<int, 5>>> py_schedule_dump(const py::dict& d, int sms) {
  return schedule_dump(gemm_desc_from(d), sms);
}

static MoeDesc moe_desc_from(const py::dict& d) {
  MoeDesc m;
  std::memset(&m, 0, sizeof(m));
  m.rank = get<int>(d, "rank", 0);
  m.R = get<int>(d, "R", 1);
  m.E = get<int>(d, "E", 0);
  m.epr = m.E / (m.R > 0 ? m.R : 1);
  m.H = get<int>(d, "H", 0);
  m.T = get<int>(d, "T", 0);
  m.topk = get<int>(d, "topk", 1);
  m.max_recv_rows = get<int>(d, "max_recv_rows", 0);
  m.bf16 = get<bool>(d, "bf16", false) ? 1 : 0;
  m.round = get<uint32_t>(d, "round", 0);
  m.tokens = reinterpret_cast<const void*>(get<int64_t>(d, "tokens", 0));
  m.topk_idx = reinterpret_cast<const int32_t*>(get<int64_t>(d, "topk_idx", 0));
  m.topk_weights = reinterpret_cast<const float*>(get<int64_t>(d, "topk_weights", 0));
  m.has_weights = m.topk_weights != nullptr ? 1 : 0;
  m.output = reinterpret_cast<void*>(get<int64_t>(d, "output", 0));
  int64_t tmp[8];
  auto fill = [&](const char* k, auto** out) {
    std::memset(tmp, 0, sizeof(tmp));
    fill_ptrs(d, k, tmp, 8);
    for (int i = 0; i < 8; ++i) out[i] = reinterpret_cast<std::remove_reference_t<decltype(out[0])>>(tmp[i]);
  };
  fill("peer_recv", m.peer_recv);
  fill("peer_out", m.peer_out);
  fill("peer_meta", m.peer_meta);
  fill("peer_meta_flags", m.peer_meta_flags);
  fill("peer_done_flags", m.peer_done_flags);
  fill("peer_ready_flags", m.peer_ready_flags);
  m.splits = reinterpret_cast<int32_t*>(get<int64_t>(d, "splits", 0));
  m.dst_row_base = reinterpret_cast<int32_t*>(get<int64_t>(d, "dst_row_base", 0));
  m.counters = reinterpret_cast<int32_t*>(get<int64_t>(d, "counters", 0));
  m.recv_seg = reinterpret_cast<int32_t*>(get<int64_t>(d, "recv_seg", 0));
  m.recv_counts = reinterpret_cast<int32_t*>(get<int64_t>(d, "recv_counts", 0));
  m.recv_total = reinterpret_cast<int32_t*>(get<int64_t>(d, "recv_total", 0));
  m.scatter_idx = reinterpret_cast<int32_t*>(get<int64_t>(d, "scatter_idx", 0));
  m.done_counter = reinterpret_cast<uint32_t*>(get<int64_t>(d, "done_counter", 0));
  m.env.status = reinterpret_cast<StatusBlock*>(get<int64_t>(d, "status_dev", 0));
  m.env.abort_word = reinterpret_cast<uint32_t*>(get<int64_t>(d, "abort_word", 0));
  {
    int64_t pa[8] = {};
    fill_ptrs(d, "peer_abort", pa, 8);
    int n = 0;
    for (int i = 0; i < 8; ++i) {
      m.env.peer_abort[i] = reinterpret_cast<uint32_t*>(pa[i]);
      if (pa[i] != 0) n = i + 1;
    }
    m.env.n_peers = static_cast<uint32_t>(n);
  }
  m.env.timeout_ns = get<uint64_t>(d, "timeout_ns", 2000000000ull);
  m.env.rank = static_cast<uint32_t>(m.rank);
  return m;
}

static torch::Tensor tensor_from_ptr(int64_t ptr, std::vector<int64_t> sizes, torch::ScalarType dt,
                                     int device) {
  auto opts = torch::TensorOptions().dtype(dt).device(torch::kCUDA, device);
  return torch::from_blob(reinterpret_cast<void*>(ptr), sizes, [](void*) {}, opts);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "tridist_b200 native runtime: symmetric heap, fused sm_100a kernels";

  // ---- symmetric heap -------------------------------------------------------
  m.def("symm_alloc", [](int64_t bytes) { return reinterpret_cast<int64_t>(symm_alloc_local(bytes)); });
  m.def("symm_free", [](int64_t p) { symm_free_local(reinterpret_cast<void*>(p)); });
  m.def("symm_export", [](int64_t p) { return py::bytes(symm_export_handle(reinterpret_cast<void*>(p))); });
  m.def("symm_open", [](py::bytes h) { return reinterpret_cast<int64_t>(symm_open_handle(std::string(h))); });
  m.def("symm_close", [](int64_t p) { symm_close_handle(reinterpret_cast<void*>(p)); });
  m.def("enable_peer_access", &symm_enable_peer_access);
  m.def("tensor_from_ptr", &tensor_from_ptr);

  // ---- virtual-memory allocations and multicast objects ------------------------------
  m.def("vmm_use_fake_driver", &vmm_use_fake_driver);
  m.def("vmm_fake_call_log", &vmm_fake_call_log);
  m.def("vmm_multicast_supported", [] {
    std::string why;
    const bool ok = vmm_multicast_supported(&why);
    return std::make_pair(ok, why);
  });
  m.def("vmm_granularity", &vmm_granularity);
  m.def("vmm_create", [](int64_t bytes) { return vmm_create(static_cast<size_t>(bytes)); });
  m.def("vmm_export_fd", &vmm_export_fd);
  m.def("vmm_import_fd", &vmm_import_fd);
  m.def("vmm_map", [](int64_t h, int64_t bytes) { return reinterpret_cast<int64_t>(vmm_map(h, static_cast<size_t>(bytes))); });
  m.def("vmm_unmap", [](int64_t p, int64_t bytes) { vmm_unmap(reinterpret_cast<void*>(p), static_cast<size_t>(bytes)); });
  m.def("vmm_release", &vmm_release);
  m.def("vmm_mc_create", [](int64_t bytes, int n) { return vmm_mc_create(static_cast<size_t>(bytes), n); });
  m.def("vmm_mc_add_device", &vmm_mc_add_device);
  m.def("vmm_mc_bind", [](int64_t mc, int64_t mem, int64_t bytes) { vmm_mc_bind(mc, mem, static_cast<size_t>(bytes)); });
  m.def("vmm_mc_unbind", [](int64_t mc, int64_t bytes) { vmm_mc_unbind(mc, static_cast<size_t>(bytes)); });

  // ---- status plane -----------------------------------------------------------
  m.def("status_alloc", [] {
    MappedStatus s = status_alloc();
    return std::make_pair(reinterpret_cast<int64_t>(s.host_ptr), reinterpret_cast<int64_t>(s.dev_ptr));
  });
  m.def("status_free", [](int64_t h) {
    status_free(MappedStatus{reinterpret_cast<StatusBlock*>(h), nullptr});
  });
  m.def("status_read", [](int64_t h) {
    const volatile uint32_t* w = reinterpret_cast<const volatile uint32_t*>(h);
    return std::vector<uint32_t>{w[0], w[1], w[2], w[3], w[4], w[5]};
  });
  m.def("status_clear", [](int64_t h) {
    volatile uint32_t* w = reinterpret_cast<volatile uint32_t*>(h);
    for (int i = 0; i < 8; ++i) w[i] = 0;
  });

  // ---- fused GEMM family --------------------------------------------------------
  m.def("gemm_plan_create", &py_gemm_plan_create);
  m.def("gemm_plan_destroy", &gemm_plan_destroy);
  m.def("gemm_plan_launch", [](int64_t id, uint32_t round, int parity, int64_t order_table, int skip_comm) {
    gemm_plan_launch(id, round, parity, order_table, skip_comm, cur_stream());
  });
  m.def("gemm_plans_launch_emulated",
        [](std::vector<int64_t> ids, uint32_t round, int parity, int skip_comm) {
          gemm_plans_launch_emulated(ids, round, parity, skip_comm, cur_stream());
        });
  m.def("launch_count", &launch_count);

  // ---- small kernels --------------------------------------------------------------
  m.def("swiglu", [](int64_t h, int64_t out, int64_t rows, int64_t inter, int64_t ldh, bool bf16) {
    swiglu_launch(reinterpret_cast<const void*>(h), reinterpret_cast<void*>(out), rows, inter, ldh, bf16,
                  cur_stream());
  });
  m.def("barrier_all", [](std::vector<int64_t> peer_slots, int rank, int R, uint32_t ticket, int64_t status_dev,
                          int64_t abort_word, uint64_t timeout_ns, std::vector<int64_t> peer_abort) {
    barrier_launch(peer_slots, rank, R, ticket, status_dev, abort_word, timeout_ns, cur_stream(), peer_abort);
  }, py::arg("peer_slots"), py::arg("rank"), py::arg("R"), py::arg("ticket"), py::arg("status_dev"),
     py::arg("abort_word"), py::arg("timeout_ns"), py::arg("peer_abort") = std::vector<int64_t>{});
  m.def("wait_flag_test", [](int64_t flag, uint32_t ticket, int64_t status_dev, int64_t abort_word,
                             uint64_t timeout_ns, std::vector<int64_t> peer_abort) {
    wait_flag_test_launch(flag, ticket, status_dev, abort_word, timeout_ns, cur_stream(), peer_abort);
  }, py::arg("flag"), py::arg("ticket"), py::arg("status_dev"), py::arg("abort_word"), py::arg("timeout_ns"),
     py::arg("peer_abort") = std::vector<int64_t>{});
  m.def("rd_exchange", [](std::vector<py::dict> blocks, int ctas, bool bf16) {
    std::vector<RdRankArgs> ranks;
    for (const auto& d : blocks) {
      RdRankArgs a{};
      a.c = reinterpret_cast<void*>(get<int64_t>(d, "c", 0));
      a.ldc = get<int64_t>(d, "ldc", 0);
      a.rows = get<int>(d, "rows", 0);
      a.n_cols = get<int>(d, "n_cols", 0);
      a.phases = get<int>(d, "phases", 0);
      a.slot = get<int>(d, "slot", 0);
      a.slots = get<int>(d, "slots", 1);
      a.flag_slices = get<int>(d, "flag_slices", kRdMaxSlices);
      a.slot_bytes = get<int64_t>(d, "slot_bytes", 0);
      a.scatter = reinterpret_cast<void*>(get<int64_t>(d, "scatter", 0));
      a.arrival = reinterpret_cast<uint32_t*>(get<int64_t>(d, "arrival", 0));
      a.ack = reinterpret_cast<uint32_t*>(get<int64_t>(d, "ack", 0));
      int64_t ps[3] = {0, 0, 0}, pa[3] = {0, 0, 0}, pk[3] = {0, 0, 0}, ab[8] = {0};
      fill_ptrs(d, "peer_scatter", ps, 3);
      fill_ptrs(d, "peer_arrival", pa, 3);
      fill_ptrs(d, "peer_ack", pk, 3);
      fill_ptrs(d, "peer_abort", ab, 8);
      for (int i = 0; i < 3; ++i) {
        a.peer_scatter[i] = reinterpret_cast<void*>(ps[i]);
        a.peer_arrival[i] = reinterpret_cast<uint32_t*>(pa[i]);
        a.peer_ack[i] = reinterpret_cast<uint32_t*>(pk[i]);
      }
      a.ticket = get<uint32_t>(d, "ticket", 0);
      a.prev_ticket = get<uint32_t>(d, "prev_ticket", 0);
      a.env.status = reinterpret_cast<StatusBlock*>(get<int64_t>(d, "status_dev", 0));
      a.env.abort_word = reinterpret_cast<uint32_t*>(get<int64_t>(d, "abort_word", 0));
      a.env.timeout_ns = get<uint64_t>(d, "timeout_ns", 4000000000ull);
      a.env.rank = get<uint32_t>(d, "rank", 0);
      for (int i = 0; i < 8; ++i)
        if (ab[i]) {
          a.env.peer_abort[i] = reinterpret_cast<uint32_t*>(ab[i]);
          a.env.n_peers = static_cast<uint32_t>(i + 1);
        }
      ranks.push_back(a);
    }
    rd_exchange_launch(ranks, ctas, bf16, cur_stream());
  }, py::arg("blocks"), py::arg("ctas"), py::arg("bf16"));
  m.def("stamp_globaltimer", [](int64_t out) { stamp_globaltimer_launch(out, cur_stream()); });
  m.def("fill_u32", [](int64_t p, int64_t n, uint32_t v) {
    fill_u32_launch(reinterpret_cast<uint32_t*>(p), n, v, cur_stream());
  });
  m.def("multimem_probe", [](int64_t mc_in, int64_t mc_out, int64_t local_out, int64_t begin, int64_t end,
                             int blocks, int threads, int unroll, bool weak, bool local_store) {
    multimem_probe_launch(mc_in, mc_out, local_out, begin, end, blocks, threads, unroll, weak, local_store,
                          cur_stream());
  });
  m.def("plan_check", &py_plan_check, py::arg("desc"), py::arg("extents"), py::arg("sms") = 148);
  m.def("schedule_dump", &py_schedule_dump, py::arg("desc"), py::arg("sms") = 148);
  m.def("splitk_dump", [](const py::dict& d, int sms) { return splitk_dump(gemm_desc_from(d), sms); },
        py::arg("desc"), py::arg("sms") = 148);
  m.def("spot_verify", [](int64_t a, int64_t b, int64_t c, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                          bool bf16, int spots, float tol, int64_t bad_tiles, int bn) {
    spot_verify_launch(a, b, c, M, N, K, lda, ldb, ldc, bf16, spots, tol, bad_tiles, bn, cur_stream());
  });

  // ---- MoE all-to-all ----------------------------------------------------------------
  m.def("moe_meta", [](const py::dict& d) { moe_meta_launch(moe_desc_from(d), cur_stream()); });
  m.def("moe_dispatch", [](const py::dict& d) { moe_dispatch_launch(moe_desc_from(d), cur_stream()); });
  m.def("moe_combine", [](const py::dict& d) { moe_combine_launch(moe_desc_from(d), cur_stream()); });
  m.def("moe_emulated", [](std::vector<py::dict> ds, int phase) {
    std::vector<MoeDesc> v;
    for (auto& d : ds) v.push_back(moe_desc_from(d));
    moe_emulated_launch(v, phase, cur_stream());
  });
}
