// Native executor of the lane pipeline of the peer-memory embedding exchange.
//
// One runtime group of a sharded table is looked up as a pipeline of lanes (sets of features that share no table row). The order
// of launches is what makes the lanes overlap - the requester half of lane i+1 in front of the owner half of lane i, the
// NVLink-bound kernels of every lane on a second ("link") stream behind an event - and with a few dozen launches per lane and
// step that order has to be issued faster than the GPU consumes it. Issued from Python, one launch costs tens of microseconds
// of interpreter, binding and allocator time; issued from here a whole forward (or backward) of all lanes is ONE call. The
// reference has nothing comparable: its exchange is four blocking torch.distributed all-to-alls per group
// (recis/nn/modules/embedding.py:498-624, recis/nn/modules/embedding_engine.py:739-801).
//
// The functions work on CUDA tensors (kernels of kernels/comm.cu, two streams) and on CPU tensors (their host twins of
// cpu/cpu_comm.cc, no streams, same order), so the multi-rank CPU tests run the very same orchestration.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include "../cpu/rb_cpu.h"
#include "../cpu/rb_cpu_comm.h"
#include "../kernels/rb_comm.h"
#include "bind_shared.h"
#include "store.h"

namespace py = pybind11;
using torch::Tensor;
using OptT = c10::optional<Tensor>;

namespace {

constexpr int kRing = 4;          // slots the per-step demand measurements come back through

RbPeers peers_of(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK(ptrs.size() <= RB_MAX_PEERS, "at most ", RB_MAX_PEERS, " ranks per node are supported by the fused exchange");
  RbPeers p;
  for (int i = 0; i < RB_MAX_PEERS; ++i) p.p[i] = i < (int)ptrs.size() ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return p;
}

// Windows, flags and counters of one lane. The memory belongs to the Python side (a symmetric heap); this object only keeps
// the tensors alive and the peer pointers at hand.
struct ExLane {
  int world = 1, rank = 0, D = 0;
  int64_t send_cap = 0, in_cap = 0;
  int64_t epoch = 0, steps = 0, last_train_epoch = 0, pending_grad_epoch = 0;
  Tensor flags, offsets, counts, ids, uemb, gin;          // this rank's views of the windows
  RbPeers p_flags, p_offsets, p_counts, p_ids, p_uemb, p_gin;
  Tensor ids_in, n_in, demand;
  Tensor ring;                                              // int32 [kRing, 2]; pinned when the lane lives on a GPU
  cudaEvent_t ring_ev[kRing] = {nullptr, nullptr, nullptr, nullptr};
  int64_t ring_step[kRing] = {-1, -1, -1, -1};
  cudaEvent_t ready_ev = nullptr;                           // "main stream has produced what the link stream needs"
  bool cuda = false;

  ExLane(int64_t world_, int64_t rank_, int64_t D_, int64_t send_cap_, int64_t in_cap_, const std::map<std::string, Tensor>& views,
         const std::map<std::string, std::vector<int64_t>>& ptrs) {
    world = (int)world_; rank = (int)rank_; D = (int)D_; send_cap = send_cap_; in_cap = in_cap_;
    flags = views.at("flags"); offsets = views.at("offsets"); counts = views.at("counts"); ids = views.at("ids");
    uemb = views.at("uemb"); gin = views.at("gin");
    p_flags = peers_of(ptrs.at("flags")); p_offsets = peers_of(ptrs.at("offsets")); p_counts = peers_of(ptrs.at("counts"));
    p_ids = peers_of(ptrs.at("ids")); p_uemb = peers_of(ptrs.at("uemb")); p_gin = peers_of(ptrs.at("gin"));
    cuda = flags.is_cuda();
    auto o = torch::TensorOptions().device(flags.device());
    ids_in = torch::empty({in_cap}, o.dtype(torch::kInt64));
    n_in = torch::zeros({1}, o.dtype(torch::kInt32));
    demand = torch::zeros({2}, o.dtype(torch::kInt32));
    ring = torch::zeros({kRing, 2}, torch::TensorOptions().dtype(torch::kInt32).pinned_memory(cuda));
    if (cuda) {
      c10::cuda::CUDAGuard g(flags.device());
      for (int i = 0; i < kRing; ++i) cudaEventCreateWithFlags(&ring_ev[i], cudaEventDisableTiming);
      cudaEventCreateWithFlags(&ready_ev, cudaEventDisableTiming);
    }
  }
  ~ExLane() {
    for (int i = 0; i < kRing; ++i) if (ring_ev[i]) cudaEventDestroy(ring_ev[i]);
    if (ready_ev) cudaEventDestroy(ready_ev);
  }
  ExLane(const ExLane&) = delete;
  ExLane& operator=(const ExLane&) = delete;

  // the device's running maxima of the window demand, copied back without anybody waiting for them
  void post_demand(cudaStream_t st) {
    const int k = (int)(steps % kRing);
    int32_t* dst = ring.data_ptr<int32_t>() + 2 * k;
    if (cuda) {
      cudaMemcpyAsync(dst, demand.data_ptr<int32_t>(), 2 * sizeof(int32_t), cudaMemcpyDeviceToHost, st);
      cudaEventRecord(ring_ev[k], st);
    } else {
      dst[0] = demand.data_ptr<int32_t>()[0]; dst[1] = demand.data_ptr<int32_t>()[1];
    }
    ring_step[k] = steps;
  }
  // (out, in) demand as measured at lookup `step` of this lane; (-1, -1) when that slot has been reused
  std::tuple<int64_t, int64_t> demand_of(int64_t step) {
    if (step < 0) return {-1, -1};
    const int k = (int)(step % kRing);
    if (ring_step[k] != step) return {-1, -1};
    if (cuda) cudaEventSynchronize(ring_ev[k]);     // issued several lookups ago: it has landed, this does not stall
    const int32_t* src = ring.data_ptr<int32_t>() + 2 * k;
    return {src[0], src[1]};
  }
};

using LanePtr = std::shared_ptr<ExLane>;

struct Ctx {
  bool cuda;
  cudaStream_t main = nullptr, link = nullptr;      // link == nullptr: everything on the main stream
  c10::optional<c10::cuda::CUDAStream> link_stream;
  Tensor status;
  int64_t wait_us;
  OptT wait_stats;
};

void wait_flags(const Ctx& c, ExLane& l, int channel, int64_t epoch, cudaStream_t st) {
  int64_t* status = c.status.data_ptr<int64_t>();
  if (!c.cuda) {
    py::gil_scoped_release nogil;          // other threads of this process (heartbeats, readers) keep running while we wait
    if (c.wait_stats.has_value() && c.wait_stats->defined())
      rbc_comm_wait_timed(l.flags.data_ptr<int64_t>(), channel, l.world, epoch, c.wait_us, status, c.wait_stats->data_ptr<int64_t>());
    else
      rbc_comm_wait(l.flags.data_ptr<int64_t>(), channel, l.world, epoch, c.wait_us, status);
    return;
  }
  if (c.wait_stats.has_value() && c.wait_stats->defined())
    rb_comm_wait_timed(l.flags.data_ptr<int64_t>(), channel, l.world, epoch, c.wait_us, status, c.wait_stats->data_ptr<int64_t>(), st);
  else
    rb_comm_wait(l.flags.data_ptr<int64_t>(), channel, l.world, epoch, c.wait_us, status, st);
}

void signal_flags(const Ctx& c, ExLane& l, int channel, int64_t epoch, cudaStream_t st) {
  if (!c.cuda) rbc_comm_signal(l.p_flags, channel, l.rank, l.world, epoch);
  else rb_comm_signal(l.p_flags, channel, l.rank, l.world, epoch, st);
}

// a tensor allocated on the main stream is about to be used on the link stream
void use_on_link(const Ctx& c, const Tensor& t) {
  if (c.link_stream.has_value() && t.defined() && t.is_cuda()) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), *c.link_stream);
}

Ctx make_ctx(const Tensor& on, Tensor status, int64_t wait_us, OptT wait_stats, int64_t link_stream) {
  Ctx c;
  c.cuda = on.is_cuda();
  c.status = status; c.wait_us = wait_us; c.wait_stats = wait_stats;
  if (c.cuda) {
    c.main = at::cuda::getCurrentCUDAStream();
    if (link_stream != 0) {
      c.link = reinterpret_cast<cudaStream_t>(link_stream);
      c.link_stream = at::cuda::getStreamFromExternal(c.link, on.device().index());
    }
  }
  return c;
}

// ---- requester half of the id phase: dedup + bucket by owner into the windows, signal IDS. Returns the reverse index.
Tensor lane_begin(const Ctx& c, ExLane& l, const Tensor& ids) {
  l.epoch += 1;
  auto r = rbx::dedup_partition(ids, l.world, l.ids, l.offsets, c.status, l.counts);
  signal_flags(c, l, RB_CH_IDS, l.epoch, c.main);
  return std::get<1>(r);
}

// ---- owner half of the id phase: ids in. Returns prefix [4*world+2] (see rb_comm_pull_ids).
Tensor lane_pull(const Ctx& c, ExLane& l, bool count_admit) {
  // With count-based admission the whole window goes through a dedup later: its tail must not hold ids of earlier steps. -2 is
  // the table's tombstone value: one ordinary dedup key that the table ignores.
  if (count_admit) l.ids_in.fill_(-2);
  wait_flags(c, l, RB_CH_IDS, l.epoch, c.main);
  auto prefix = torch::empty({4 * l.world + 2}, l.n_in.options());
  if (!c.cuda) {
    rbc_comm_pull_ids(l.p_ids, l.p_offsets, l.p_counts, l.rank, l.world, l.ids_in.data_ptr<int64_t>(), l.in_cap, prefix.data_ptr<int32_t>(),
                      l.n_in.data_ptr<int32_t>(), l.demand.data_ptr<int32_t>(), c.status.data_ptr<int64_t>());
  } else {
    rb_comm_pull_ids(l.p_ids, l.p_offsets, l.p_counts, l.rank, l.world, l.ids_in.data_ptr<int64_t>(), l.in_cap, prefix.data_ptr<int32_t>(),
                     l.n_in.data_ptr<int32_t>(), l.demand.data_ptr<int32_t>(), c.status.data_ptr<int64_t>(), c.main);
  }
  l.post_demand(c.main);
  l.steps += 1;
  return prefix;
}

Tensor lane_lookup(ExLane& l, rbx::EmbeddingStore& store, bool readonly, int64_t threshold, const OptT& step) {
  if (readonly) return store.find(l.ids_in, l.n_in);
  if (threshold > 1) {
    // count-based admission counts ONE sighting per id and step, whoever asks: dedup the incoming ids before the table sees them
    auto d = rbx::dedup_partition(l.ids_in, 1, c10::nullopt, c10::nullopt, c10::nullopt, c10::nullopt);
    auto o_rows = store.lookup_or_insert(std::get<0>(d), std::get<3>(d).narrow(0, 1, 1), step, threshold, /*ids_unique=*/true);
    return o_rows.index_select(0, std::get<1>(d).to(torch::kInt64)).contiguous();
  }
  return store.lookup_or_insert(l.ids_in, l.n_in, step, threshold);
}

// ---- owner: push the rows to the requesters (link stream when there is one), signal EMB
void lane_push(const Ctx& c, ExLane& l, const Tensor& emb, const Tensor& rows_in, const Tensor& prefix, int64_t blocks) {
  if (!c.cuda) {
    rbc_comm_push_emb(emb.data_ptr(), rows_in.data_ptr<int32_t>(), prefix.data_ptr<int32_t>(), l.p_uemb, l.rank, l.world,
                      (int64_t)l.D * emb.element_size(), l.in_cap);
    rbc_comm_signal(l.p_flags, RB_CH_EMB, l.rank, l.world, l.epoch);
    return;
  }
  cudaStream_t st = c.main;
  if (c.link != nullptr) {
    cudaEventRecord(l.ready_ev, c.main);
    cudaStreamWaitEvent(c.link, l.ready_ev, 0);
    use_on_link(c, rows_in); use_on_link(c, prefix);
    st = c.link;
  }
  rb_comm_push_emb(emb.data_ptr(), rows_in.data_ptr<int32_t>(), prefix.data_ptr<int32_t>(), l.p_uemb, l.rank, l.world,
                   (int64_t)l.D * emb.element_size(), l.in_cap, c.link != nullptr ? (int)blocks : 0, st);
  rb_comm_signal(l.p_flags, RB_CH_EMB, l.rank, l.world, l.epoch, st);
}

// Lookup of one runtime group split into lanes; see FusedExchange.forward_group for the layout arguments. Returns the shared
// output [n_rows, D] and, per lane, (rev, gsrc, gscale, rows_in, prefix, epoch as a 0-dim tensor is avoided: epochs come back
// as a separate list).
std::tuple<Tensor, std::vector<std::vector<Tensor>>, std::vector<int64_t>> exchange_forward_group(
    std::vector<LanePtr> lanes, std::shared_ptr<rbx::EmbeddingStore> store, std::vector<Tensor> ids, std::vector<Tensor> offsets,
    std::vector<OptT> weights, std::vector<int64_t> perm_f, std::vector<int64_t> perm_off, int64_t mode, int64_t perm_b,
    int64_t perm_total, int64_t n_rows, bool train, bool readonly, int64_t threshold, OptT step, Tensor status, int64_t wait_us,
    OptT wait_stats, int64_t link_stream, int64_t push_blocks) {
  const size_t L = lanes.size();
  TORCH_CHECK(L >= 1 && ids.size() == L && offsets.size() == L && weights.size() == L && perm_f.size() == L && perm_off.size() == L);
  ExLane& l0 = *lanes[0];
  c10::cuda::OptionalCUDAGuard guard;
  if (l0.cuda) guard.set_device(l0.flags.device());
  Ctx c = make_ctx(l0.flags, status, wait_us, wait_stats, L > 1 ? link_stream : 0);
  const int D = l0.D;
  const bool count_admit = !readonly && threshold > 1;
  auto out = torch::empty({n_rows, D}, torch::TensorOptions().dtype(torch::kFloat32).device(l0.flags.device()));
  std::vector<Tensor> rev(L), rows_in(L), prefix(L);
  Tensor emb = store->emb();
  TORCH_CHECK(emb.scalar_type() == l0.uemb.scalar_type(), "the exchange windows carry ", l0.uemb.scalar_type(), " rows, the table stores ", emb.scalar_type());
  rev[0] = lane_begin(c, *lanes[0], ids[0]);
  for (size_t i = 0; i < L; ++i) {
    if (i + 1 < L) rev[i + 1] = lane_begin(c, *lanes[i + 1], ids[i + 1]);     // the next lane's ids are on offer before this lane waits
    prefix[i] = lane_pull(c, *lanes[i], count_admit);
    rows_in[i] = lane_lookup(*lanes[i], *store, readonly, threshold, step);
    emb = store->emb();                                                     // the arena may have grown
    lane_push(c, *lanes[i], emb, rows_in[i], prefix[i], push_blocks);
  }
  std::vector<std::vector<Tensor>> saved;
  std::vector<int64_t> epochs;
  for (size_t i = 0; i < L; ++i) {
    ExLane& l = *lanes[i];
    wait_flags(c, l, RB_CH_EMB, l.epoch, c.main);
    const int64_t n_seg = offsets[i].numel() - 1, n = rev[i].numel();
    Tensor gsrc, gscale;
    if (train) { gsrc = torch::empty({n}, rev[i].options()); gscale = torch::empty({n}, out.options()); }
    const float* wp = weights[i].has_value() && weights[i]->defined() ? weights[i]->data_ptr<float>() : nullptr;
    const int pb = perm_total > 0 ? (int)perm_b : 0, pf = perm_total > 0 ? (int)perm_f[i] : 0;
    if (pf > 0) {
      TORCH_CHECK((int64_t)pb * pf == n_seg && perm_off[i] + pf <= perm_total && n_rows == (int64_t)pb * perm_total, "lane layout does not match its segments");
    } else {
      TORCH_CHECK(perm_off[i] + n_seg <= n_rows, "lane rows exceed the shared output");
    }
    if (!c.cuda) {
      rbc_pool_forward(l.uemb.data_ptr(), rbx::row_dtype_of(l.uemb), nullptr, rev[i].data_ptr<int32_t>(), offsets[i].data_ptr<int32_t>(), wp, n_seg, D, (int)mode, pb,
                       pf, (int)perm_off[i], (int)perm_total, out.data_ptr<float>(), train ? gsrc.data_ptr<int32_t>() : nullptr,
                       train ? gscale.data_ptr<float>() : nullptr);
    } else {
      rb_pool_forward(l.uemb.data_ptr(), rbx::row_dtype_of(l.uemb), nullptr, rev[i].data_ptr<int32_t>(), offsets[i].data_ptr<int32_t>(), wp, n_seg, D, (int)mode, pb,
                      pf, (int)perm_off[i], (int)perm_total, out.data_ptr<float>(), train ? gsrc.data_ptr<int32_t>() : nullptr,
                      train ? gscale.data_ptr<float>() : nullptr, c.main);
    }
    if (train) {
      l.last_train_epoch = l.epoch;
      saved.push_back({rev[i], gsrc, gscale, rows_in[i], prefix[i]});
      epochs.push_back(l.epoch);
    }
  }
  return {out, saved, epochs};
}

// Backward of exchange_forward_group: per lane, the element sort on the main stream, the NVLink-bound reduce + push on the
// link stream behind an event, then the GRAD signal. saved[i] = (rev, gsrc, gscale, rows_in, prefix).
void exchange_backward_group(std::vector<LanePtr> lanes, std::vector<std::vector<Tensor>> saved, std::vector<int64_t> epochs,
                             const Tensor& grad_out, Tensor status, int64_t link_stream, int64_t max_blocks) {
  const size_t L = lanes.size();
  TORCH_CHECK(saved.size() == L && epochs.size() == L);
  TORCH_CHECK(grad_out.is_contiguous() && grad_out.scalar_type() == torch::kFloat32, "grad_out must be contiguous fp32");
  ExLane& l0 = *lanes[0];
  c10::cuda::OptionalCUDAGuard guard;
  if (l0.cuda) guard.set_device(l0.flags.device());
  Ctx c = make_ctx(l0.flags, status, 0, c10::nullopt, L > 1 ? link_stream : 0);
  const int D = l0.D, W = l0.world;
  use_on_link(c, grad_out);
  for (size_t i = 0; i < L; ++i) {
    ExLane& l = *lanes[i];
    const Tensor &rev = saved[i][0], &gsrc = saved[i][1], &gscale = saved[i][2], &prefix = saved[i][4];
    auto csr = rbx::build_csr(rev);
    const Tensor &csr_u = std::get<0>(csr), &csr_elem = std::get<1>(csr), &start = std::get<2>(csr);
    const int32_t* off = prefix.data_ptr<int32_t>() + 3 * W + 1;            // this rank's own bucket boundaries of that step
    const int32_t* dst_base = prefix.data_ptr<int32_t>() + 2 * W + 1;
    const int64_t n = csr_u.numel();
    if (!c.cuda) {
      const int64_t n_u = off[W];
      auto gu = torch::zeros({std::max<int64_t>(n_u, 1), D}, grad_out.options());
      RbOpt none{};
      none.kind = RB_OPT_SGD; none.grad_scale = 1.f; none.decay = 1.f; none.w_dtype = 0;
      if (n > 0)
        rbc_grad_reduce(grad_out.data_ptr<float>(), gsrc.data_ptr<int32_t>(), gscale.data_ptr<float>(), csr_u.data_ptr<int32_t>(),
                        csr_elem.data_ptr<int32_t>(), start.data_ptr<int32_t>(), n, D, nullptr, gu.data_ptr<float>(), 0, none);
      rbc_comm_push_grads(gu.data_ptr<float>(), D, off, dst_base, l.p_gin, W, l.in_cap);
      rbc_comm_signal(l.p_flags, RB_CH_GRAD, l.rank, W, epochs[i]);
      continue;
    }
    cudaStream_t st = c.main;
    if (c.link != nullptr) {
      cudaEventRecord(l.ready_ev, c.main);
      cudaStreamWaitEvent(c.link, l.ready_ev, 0);
      for (const Tensor& t : {csr_u, csr_elem, start, gsrc, gscale, prefix}) use_on_link(c, t);
      st = c.link;
    }
    if (n > 0) {
      RbGuPush push{};
      push.off = off; push.dst_base = dst_base;
      for (int r = 0; r < W; ++r) push.base[r] = l.p_gin.p[r];
      push.world = W; push.cap_rows = l.in_cap;
      const int64_t n_chunks = (n + rb_grad_reduce_chunk() - 1) / rb_grad_reduce_chunk();
      Tensor span;
      {
        // allocated and zeroed on the stream that uses it
        c10::cuda::OptionalCUDAStreamGuard sg;
        if (c.link != nullptr) sg.reset_stream(*c.link_stream);
        span = torch::zeros({n_chunks, D}, grad_out.options());
      }
      rb_grad_reduce_push(grad_out.data_ptr<float>(), gsrc.data_ptr<int32_t>(), gscale.data_ptr<float>(), csr_u.data_ptr<int32_t>(),
                          csr_elem.data_ptr<int32_t>(), start.data_ptr<int32_t>(), n, D, span.data_ptr<float>(), push,
                          c.link != nullptr ? (int)max_blocks : 0, st);
    }
    rb_comm_signal(l.p_flags, RB_CH_GRAD, l.rank, W, epochs[i], st);
  }
}

}  // namespace

void init_exchange(py::module& m) {
  py::class_<ExLane, LanePtr>(m, "ExLane")
      .def(py::init<int64_t, int64_t, int64_t, int64_t, int64_t, const std::map<std::string, Tensor>&,
                    const std::map<std::string, std::vector<int64_t>>&>())
      .def_readwrite("epoch", &ExLane::epoch)
      .def_readwrite("steps", &ExLane::steps)
      .def_readwrite("last_train_epoch", &ExLane::last_train_epoch)
      .def_readwrite("pending_grad_epoch", &ExLane::pending_grad_epoch)
      .def_readonly("send_cap", &ExLane::send_cap)
      .def_readonly("in_cap", &ExLane::in_cap)
      .def_readonly("ids_in", &ExLane::ids_in)
      .def_readonly("n_in", &ExLane::n_in)
      .def_readonly("demand", &ExLane::demand)
      .def("post_demand", [](ExLane& l) { l.post_demand(l.cuda ? (cudaStream_t)at::cuda::getCurrentCUDAStream() : nullptr); })
      .def("demand_of", &ExLane::demand_of);
  m.def("exchange_forward_group", &exchange_forward_group);
  m.def("exchange_backward_group", &exchange_backward_group);
}
