// pybind11 bindings of the host-only C++ (no CUDA, no torch): Belady planner, file tier, CPU
// reference attention. Arrays cross as NumPy buffers.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "cpu_ref/flash_cpu.h"
#include "cpu_ref/quant_adamw_ref.h"
#include "attn/tile_iter_host.h"
#include "peer/barrier_model.h"
#include "tier/belady_min.h"
#include "tier/tier_engine.h"

namespace py = pybind11;
using namespace zxh;

namespace {

py::dict result_to_dict(const BeladyResult& r) {
  py::dict d;
  d["hit"] = py::array_t<uint8_t>((py::ssize_t)r.hit.size(), r.hit.data());
  d["next_use"] = py::array_t<int64_t>((py::ssize_t)r.next_use.size(), r.next_use.data());
  d["evicted"] = r.evicted;
  d["hits"] = r.hits;
  d["misses"] = r.misses;
  d["bytes_loaded"] = r.bytes_loaded;
  d["bytes_evicted"] = r.bytes_evicted;
  d["peak_resident_bytes"] = r.peak_resident_bytes;
  d["bypassed"] = r.bypassed;
  return d;
}

using FArr = py::array_t<float, py::array::c_style | py::array::forcecast>;
using IArr = py::array_t<int64_t, py::array::c_style | py::array::forcecast>;

CpuAttnShape shape_of(const FArr& q, const FArr& k, float scale, bool causal, int wb, int ge) {
  if (q.ndim() != 4 || k.ndim() != 4) throw std::runtime_error("flash_cpu: q and k must be [B,S,H,D]");
  CpuAttnShape s;
  s.B = (int)q.shape(0); s.Sq = (int)q.shape(1); s.Hq = (int)q.shape(2); s.D = (int)q.shape(3);
  s.Skv = (int)k.shape(1); s.Hkv = (int)k.shape(2);
  if (s.Hq % s.Hkv != 0) throw std::runtime_error("flash_cpu: Hq must be a multiple of Hkv");
  s.scale = scale; s.causal = causal; s.window_blocks = wb; s.global_every = ge;
  return s;
}

}  // namespace

PYBIND11_MODULE(_host, m) {
  m.def("quant_e4m3_ref", [](py::array_t<float, py::array::c_style | py::array::forcecast> x, int block_tokens) {
    if (x.ndim() != 3) throw std::runtime_error("quant_e4m3_ref: x must be [tokens, heads, dim]");
    const int64_t tokens = x.shape(0);
    const int heads = (int)x.shape(1), dim = (int)x.shape(2);
    py::array_t<uint8_t> q({(py::ssize_t)tokens, (py::ssize_t)heads, (py::ssize_t)dim});
    py::array_t<float> sc({(py::ssize_t)((tokens + block_tokens - 1) / block_tokens), (py::ssize_t)heads});
    zx::quant_e4m3_ref(x.data(), q.mutable_data(), sc.mutable_data(), tokens, heads, dim, block_tokens);
    return py::make_tuple(q, sc);
  }, py::arg("x"), py::arg("block_tokens") = 128);
  m.def("e4m3_to_float", [](py::array_t<uint8_t, py::array::c_style | py::array::forcecast> q) {
    py::array_t<float> out(q.size());
    for (py::ssize_t i = 0; i < q.size(); ++i) out.mutable_data()[i] = zx::e4m3_to_float(q.data()[i]);
    return out;
  });
  m.def("adamw_split_master_ref", [](py::array_t<uint16_t, py::array::c_style> p_hi, py::array_t<int16_t, py::array::c_style> p_lo,
                                     py::array_t<float, py::array::c_style> mm, py::array_t<float, py::array::c_style> vv,
                                     py::array_t<float, py::array::c_style | py::array::forcecast> g, size_t decay_end, float lr,
                                     float beta1, float beta2, float eps, float weight_decay, int step) {
    const size_t n = (size_t)p_hi.size();
    if ((size_t)p_lo.size() != n || (size_t)mm.size() != n || (size_t)vv.size() != n || (size_t)g.size() != n)
      throw std::runtime_error("adamw_split_master_ref: size mismatch");
    zx::adamw_split_master_ref(p_hi.mutable_data(), p_lo.mutable_data(), mm.mutable_data(), vv.mutable_data(), g.data(), n,
                               decay_end, lr, beta1, beta2, eps, weight_decay, step);
  }, "in place on p_hi (bf16 bits), p_lo, m, v");

  m.def("tile_iter_mismatches", &zx::tile_iter_mismatches, py::arg("causal"), py::arg("window_blocks"),
        py::arg("global_every"), py::arg("q_chunk_pos"), py::arg("kv_chunk_pos"), py::arg("q_tiles_per_chunk"),
        py::arg("kv_tiles_per_chunk"));
  m.def("barrier_model", [](int ranks, int rounds, uint32_t start_epoch, uint64_t seed, int absent_rank,
                            int absent_from_round, int64_t timeout_us) {
    zx::BarrierModelResult r;
    {
      py::gil_scoped_release nogil;
      r = zx::run_barrier_model(ranks, rounds, start_epoch, seed, absent_rank, absent_from_round, timeout_us);
    }
    py::dict d;
    d["violations"] = r.violations;
    d["timeouts"] = r.timeouts;
    d["rounds_done"] = r.rounds_done;
    return d;
  }, py::arg("ranks"), py::arg("rounds"), py::arg("start_epoch") = 0, py::arg("seed") = 0, py::arg("absent_rank") = -1,
     py::arg("absent_from_round") = 0, py::arg("timeout_us") = 2000000);
  m.def("belady_min", [](const std::vector<int64_t>& ids, const std::vector<int64_t>& size_of, int64_t cap) {
    for (auto id : ids)
      if (id < 0 || id >= (int64_t)size_of.size()) throw std::runtime_error("belady_min: block id out of range");
    return result_to_dict(belady_min(ids, size_of, cap));
  });
  m.def("lru_trace", [](const std::vector<int64_t>& ids, const std::vector<int64_t>& size_of, int64_t cap) {
    for (auto id : ids)
      if (id < 0 || id >= (int64_t)size_of.size()) throw std::runtime_error("lru_trace: block id out of range");
    return result_to_dict(lru_trace(ids, size_of, cap));
  });

  py::class_<FileTier>(m, "FileTier")
      .def(py::init<const std::string&, int64_t, int64_t, int, bool>(), py::arg("path"), py::arg("slot_bytes"),
           py::arg("num_slots"), py::arg("num_threads") = 2, py::arg("try_direct") = true)
      .def("write_async", [](FileTier& t, int64_t slot, int64_t ptr, int64_t bytes) {
        return t.write_async(slot, reinterpret_cast<const void*>(ptr), bytes);
      })
      .def("read_async", [](FileTier& t, int64_t slot, int64_t ptr, int64_t bytes) {
        return t.read_async(slot, reinterpret_cast<void*>(ptr), bytes);
      })
      .def("wait", [](FileTier& t, int64_t ticket) {
        py::gil_scoped_release rel;
        return t.wait(ticket);
      })
      .def("wait_all", [](FileTier& t) {
        py::gil_scoped_release rel;
        t.wait_all();
      })
      .def_property_readonly("direct", &FileTier::direct)
      .def_property_readonly("bytes_written", &FileTier::bytes_written)
      .def_property_readonly("bytes_read", &FileTier::bytes_read);

  m.def("flash_cpu_forward", [](FArr q, FArr k, FArr v, IArr qpos, IArr kpos, float scale, bool causal, int wb, int ge,
                                py::object o_prev, py::object lse_prev) {
    CpuAttnShape s = shape_of(q, k, scale, causal, wb, ge);
    const bool merge = !o_prev.is_none();
    FArr o = merge ? FArr(o_prev.cast<FArr>().request()) : FArr({s.B, s.Sq, s.Hq, s.D});
    FArr lse = merge ? FArr(lse_prev.cast<FArr>().request()) : FArr({s.B, s.Hq, s.Sq});
    {
      py::gil_scoped_release rel;
      flash_cpu_forward(s, q.data(), k.data(), v.data(), qpos.data(), kpos.data(), o.mutable_data(),
                        lse.mutable_data(), merge);
    }
    return py::make_tuple(o, lse);
  }, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("qpos"), py::arg("kpos"), py::arg("scale"),
     py::arg("causal") = true, py::arg("window_blocks") = 0, py::arg("global_every") = 0,
     py::arg("o_prev") = py::none(), py::arg("lse_prev") = py::none());

  m.def("flash_cpu_backward", [](FArr q, FArr k, FArr v, FArr o, FArr d_o, FArr lse, IArr qpos, IArr kpos, float scale,
                                 bool causal, int wb, int ge) {
    CpuAttnShape s = shape_of(q, k, scale, causal, wb, ge);
    FArr dq({s.B, s.Sq, s.Hq, s.D}), dk({s.B, s.Skv, s.Hkv, s.D}), dv({s.B, s.Skv, s.Hkv, s.D});
    std::fill(dk.mutable_data(), dk.mutable_data() + dk.size(), 0.f);
    std::fill(dv.mutable_data(), dv.mutable_data() + dv.size(), 0.f);
    {
      py::gil_scoped_release rel;
      flash_cpu_backward(s, q.data(), k.data(), v.data(), o.data(), d_o.data(), lse.data(), qpos.data(), kpos.data(),
                         dq.mutable_data(), dk.mutable_data(), dv.mutable_data());
    }
    return py::make_tuple(dq, dk, dv);
  }, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("o"), py::arg("d_o"), py::arg("lse"), py::arg("qpos"),
     py::arg("kpos"), py::arg("scale"), py::arg("causal") = true, py::arg("window_blocks") = 0,
     py::arg("global_every") = 0);
}
