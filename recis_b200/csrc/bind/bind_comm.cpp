// Symmetric (peer-mapped) memory and the Python bindings of the peer-memory exchange kernels.
//
// A symmetric buffer is a plain cudaMalloc allocation (outside torch's caching allocator, so that it can be exported)
// wrapped as a tensor; its cudaIpc handle is exchanged through torch.distributed by the Python side and opened by every
// other rank. Kernels then receive one pointer per rank. The reference has nothing comparable: all of its inter-GPU
// traffic goes through torch.distributed collectives (recis/nn/modules/embedding.py:73-118,498-542).
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <unistd.h>
#include "../cpu/rb_cpu.h"
#include "../cpu/rb_cpu_comm.h"
#include "../kernels/rb_comm.h"
#include "store.h"
#include "bind_shared.h"

namespace py = pybind11;
using torch::Tensor;
using OptT = c10::optional<Tensor>;

namespace {

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream(); }

#define RB_CUDA_CHECK(expr)                                                                         \
  do {                                                                                              \
    cudaError_t e__ = (expr);                                                                       \
    TORCH_CHECK(e__ == cudaSuccess, #expr, " failed: ", cudaGetErrorString(e__));                   \
  } while (0)

// (tensor over a fresh zeroed cudaMalloc allocation, its 64-byte IPC handle)
std::tuple<Tensor, py::bytes> sym_alloc(int64_t nbytes, int64_t device_index) {
  c10::cuda::CUDAGuard g(torch::Device(torch::kCUDA, (c10::DeviceIndex)device_index));
  void* ptr = nullptr;
  nbytes = std::max<int64_t>((nbytes + 255) / 256 * 256, 256);
  RB_CUDA_CHECK(cudaMalloc(&ptr, (size_t)nbytes));
  RB_CUDA_CHECK(cudaMemset(ptr, 0, (size_t)nbytes));
  cudaIpcMemHandle_t h;
  RB_CUDA_CHECK(cudaIpcGetMemHandle(&h, ptr));
  auto t = torch::from_blob(ptr, {nbytes}, [](void* p) { cudaFree(p); },
                            torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA, (c10::DeviceIndex)device_index));
  return {t, py::bytes(reinterpret_cast<const char*>(&h), sizeof(h))};
}

int64_t sym_open(const std::string& handle, int64_t device_index) {
  TORCH_CHECK(handle.size() == sizeof(cudaIpcMemHandle_t), "bad IPC handle size");
  c10::cuda::CUDAGuard g(torch::Device(torch::kCUDA, (c10::DeviceIndex)device_index));
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle.data(), sizeof(h));
  void* ptr = nullptr;
  RB_CUDA_CHECK(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return reinterpret_cast<int64_t>(ptr);
}

void sym_close(int64_t ptr) { cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)); }

// ---- host twin of the symmetric heap: a POSIX shared-memory object per rank, mapped by every rank of the node
// (zero-filled tensor over a fresh shared-memory object called `name`; the object is unlinked when the tensor dies)
Tensor shm_alloc(const std::string& name, int64_t nbytes) {
  nbytes = std::max<int64_t>((nbytes + 4095) / 4096 * 4096, 4096);
  const int fd = shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
  TORCH_CHECK(fd >= 0, "shm_open(", name, ") failed: ", std::strerror(errno));
  if (ftruncate(fd, nbytes) != 0) { const int e = errno; close(fd); shm_unlink(name.c_str()); TORCH_CHECK(false, "ftruncate failed: ", std::strerror(e)); }
  void* ptr = mmap(nullptr, (size_t)nbytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (ptr == MAP_FAILED) { shm_unlink(name.c_str()); TORCH_CHECK(false, "mmap failed: ", std::strerror(errno)); }
  std::memset(ptr, 0, (size_t)nbytes);
  return torch::from_blob(ptr, {nbytes}, [name, nbytes](void* p) { munmap(p, (size_t)nbytes); shm_unlink(name.c_str()); },
                          torch::TensorOptions().dtype(torch::kUInt8));
}

// maps a peer's object; returns (address, mapped bytes) for shm_close
std::tuple<int64_t, int64_t> shm_open_peer(const std::string& name) {
  const int fd = shm_open(name.c_str(), O_RDWR, 0600);
  TORCH_CHECK(fd >= 0, "shm_open(", name, ") failed: ", std::strerror(errno));
  const off_t nbytes = lseek(fd, 0, SEEK_END);
  void* ptr = mmap(nullptr, (size_t)nbytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  TORCH_CHECK(ptr != MAP_FAILED, "mmap failed: ", std::strerror(errno));
  return {reinterpret_cast<int64_t>(ptr), (int64_t)nbytes};
}

void shm_close(int64_t ptr, int64_t nbytes) { munmap(reinterpret_cast<void*>(ptr), (size_t)nbytes); }

// removes the name; the memory lives on until the last mapping goes (called once every rank has mapped it, so that a rank
// that dies later leaves nothing behind in the shared-memory directory)
void shm_unlink_name(const std::string& name) { shm_unlink(name.c_str()); }

RbPeers peers_of(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK(ptrs.size() <= RB_MAX_PEERS, "at most ", RB_MAX_PEERS, " ranks per node are supported by the fused exchange");
  RbPeers p;
  for (int i = 0; i < RB_MAX_PEERS; ++i) p.p[i] = i < (int)ptrs.size() ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return p;
}

// host = true: the pads are shared-memory mappings and the stores are done by this thread
void comm_signal(const std::vector<int64_t>& flag_pads, int64_t channel, int64_t me, int64_t epoch, bool host) {
  if (host) { rbc_comm_signal(peers_of(flag_pads), (int)channel, (int)me, (int)flag_pads.size(), epoch); return; }
  rb_comm_signal(peers_of(flag_pads), (int)channel, (int)me, (int)flag_pads.size(), epoch, cur_stream());
}

void comm_wait(const Tensor& flags, int64_t channel, int64_t world, int64_t epoch, int64_t spin_limit, Tensor status) {
  if (!flags.is_cuda()) {
    py::gil_scoped_release nogil;           // other threads of this process (heartbeats, readers) keep running while we wait
    rbc_comm_wait(flags.data_ptr<int64_t>(), (int)channel, (int)world, epoch, spin_limit, status.data_ptr<int64_t>());
    return;
  }
  rb_comm_wait(flags.data_ptr<int64_t>(), (int)channel, (int)world, epoch, spin_limit, status.data_ptr<int64_t>(), cur_stream());
}

// peer_counts: the requesters' unclamped per-owner unique counts (may be empty); demand: int32[2] running maxima (may be undefined)
void comm_pull_ids(const std::vector<int64_t>& peer_ids, const std::vector<int64_t>& peer_offsets, const std::vector<int64_t>& peer_counts,
                   int64_t me, Tensor ids_in, Tensor prefix, Tensor n_in, OptT demand, Tensor status) {
  const int world = (int)peer_ids.size();
  TORCH_CHECK(prefix.numel() >= 4 * world + 2 && prefix.scalar_type() == torch::kInt32, "prefix: int32 [4 * world + 2]");
  RbPeers counts = peers_of(peer_counts);
  int32_t* dm = demand.has_value() && demand->defined() ? demand->data_ptr<int32_t>() : nullptr;
  if (!ids_in.is_cuda()) {
    rbc_comm_pull_ids(peers_of(peer_ids), peers_of(peer_offsets), counts, (int)me, world, ids_in.data_ptr<int64_t>(), ids_in.numel(),
                      prefix.data_ptr<int32_t>(), n_in.data_ptr<int32_t>(), dm, status.data_ptr<int64_t>());
    return;
  }
  c10::cuda::CUDAGuard g(ids_in.device());
  rb_comm_pull_ids(peers_of(peer_ids), peers_of(peer_offsets), counts, (int)me, world, ids_in.data_ptr<int64_t>(), ids_in.numel(),
                   prefix.data_ptr<int32_t>(), n_in.data_ptr<int32_t>(), dm, status.data_ptr<int64_t>(), cur_stream());
}

void comm_push_emb(const Tensor& emb, const Tensor& rows_in, const Tensor& prefix, const std::vector<int64_t>& peer_uemb, int64_t me,
                   int64_t n_in_hint, int64_t blocks) {
  const int64_t row_bytes = emb.size(1) * emb.element_size();
  if (!emb.is_cuda()) {
    rbc_comm_push_emb(emb.data_ptr(), rows_in.data_ptr<int32_t>(), prefix.data_ptr<int32_t>(), peers_of(peer_uemb), (int)me,
                      (int)peer_uemb.size(), row_bytes, n_in_hint);
    return;
  }
  TORCH_CHECK(row_bytes % 16 == 0, "the fused exchange needs rows that are a multiple of 16 bytes");
  c10::cuda::CUDAGuard g(emb.device());
  rb_comm_push_emb(emb.data_ptr(), rows_in.data_ptr<int32_t>(), prefix.data_ptr<int32_t>(), peers_of(peer_uemb), (int)me,
                   (int)peer_uemb.size(), row_bytes, n_in_hint, (int)blocks, cur_stream());
}

// apply: update rows of (w, s1, s2) in place. Otherwise returns (rows [n_in_max] with -1 holes, grads [n_in_max, D]).
std::tuple<Tensor, Tensor> comm_owner_reduce(const Tensor& rows_in, Tensor head, const Tensor& prefix, const Tensor& g_in, int64_t world, int64_t D, bool mean_by_id, bool apply,
                                             int64_t kind, double lr, double beta1, double beta2, double eps, double decay, double alpha,
                                             double grad_scale, OptT w, OptT s1, OptT s2, int64_t n_in_hint, int64_t unroll) {
  RbOpt o = rbx::make_opt(kind, lr, beta1, beta2, eps, decay, alpha, grad_scale, w, s1, s2);
  const int64_t n_max = rows_in.numel();
  auto next = torch::empty({n_max}, rows_in.options());
  Tensor out_rows, out_grads;
  if (!apply) {
    out_rows = torch::full({n_in_hint}, -1, rows_in.options());
    out_grads = torch::zeros({n_in_hint, D}, rows_in.options().dtype(torch::kFloat32));
  } else {
    TORCH_CHECK(o.w != nullptr, "apply needs the weight slab");
  }
  if (!rows_in.is_cuda()) {
    rbc_comm_owner_reduce(rows_in.data_ptr<int32_t>(), head.data_ptr<int32_t>(), next.data_ptr<int32_t>(), prefix.data_ptr<int32_t>(),
                          g_in.data_ptr<float>(), (int)world, (int)D, mean_by_id, apply, o, apply ? nullptr : out_rows.data_ptr<int32_t>(),
                          apply ? nullptr : out_grads.data_ptr<float>());
    return {out_rows, out_grads};
  }
  rb_comm_owner_reduce(rows_in.data_ptr<int32_t>(), head.data_ptr<int32_t>(), next.data_ptr<int32_t>(), prefix.data_ptr<int32_t>(),
                       g_in.data_ptr<float>(), (int)world, (int)D, mean_by_id, apply, o,
                       apply ? nullptr : out_rows.data_ptr<int32_t>(), apply ? nullptr : out_grads.data_ptr<float>(), n_in_hint,
                       (int)unroll, cur_stream());
  return {out_rows, out_grads};
}

// Requester side of the backward exchange: reduce the pooled gradient to one gradient per unique id and store each of
// them straight into the window of the rank that owns the id (peer stores). offsets = this rank's bucket boundaries
// [world+1]; meta = the tensor written by comm_pull_ids (the destination bases sit at meta[2*world+1 ..]).
void comm_grad_reduce_push(const Tensor& grad_out, const Tensor& gsrc, const Tensor& gscale, const Tensor& csr_u, const Tensor& csr_elem,
                           const Tensor& start, int64_t D, const Tensor& offsets, const Tensor& meta,
                           const std::vector<int64_t>& peer_gin, int64_t cap_rows, int64_t max_blocks) {
  if (!grad_out.is_cuda()) {
    // host twin: per-unique gradients first (the CPU reduction), then one row copy per unique id into its owner's window
    TORCH_CHECK(grad_out.is_contiguous() && grad_out.scalar_type() == torch::kFloat32, "grad_out must be contiguous fp32");
    const int world = (int)peer_gin.size();
    const int32_t* off = offsets.data_ptr<int32_t>();
    const int64_t n_u = off[world];
    auto gu = torch::zeros({std::max<int64_t>(n_u, 1), D}, grad_out.options());
    RbOpt none{};
    none.kind = RB_OPT_SGD; none.grad_scale = 1.f; none.decay = 1.f; none.w_dtype = 0;
    if (csr_u.numel() > 0)
      rbc_grad_reduce(grad_out.data_ptr<float>(), gsrc.data_ptr<int32_t>(), gscale.data_ptr<float>(), csr_u.data_ptr<int32_t>(),
                      csr_elem.data_ptr<int32_t>(), start.data_ptr<int32_t>(), csr_u.numel(), (int)D, nullptr, gu.data_ptr<float>(), 0, none);
    RbPeers peers = peers_of(peer_gin);
    rbc_comm_push_grads(gu.data_ptr<float>(), (int)D, off, meta.data_ptr<int32_t>() + 2 * world + 1, peers, world, cap_rows);
    return;
  }
  TORCH_CHECK(grad_out.is_cuda() && grad_out.is_contiguous() && grad_out.scalar_type() == torch::kFloat32, "grad_out must be contiguous fp32 on CUDA");
  TORCH_CHECK(D % 4 == 0 && D <= 512, "the fused exchange needs an embedding width that is a multiple of 4 and at most 512");
  const int64_t n = csr_u.numel();
  if (n == 0) return;
  const int world = (int)peer_gin.size();
  TORCH_CHECK(world <= RB_MAX_PEERS && offsets.numel() >= world + 1 && meta.numel() >= 3 * world + 1);
  c10::cuda::CUDAGuard g(grad_out.device());
  RbGuPush push{};
  push.off = offsets.data_ptr<int32_t>();
  push.dst_base = meta.data_ptr<int32_t>() + 2 * world + 1;
  for (int r = 0; r < world; ++r) push.base[r] = reinterpret_cast<void*>(peer_gin[r]);
  push.world = world;
  push.cap_rows = cap_rows;
  const int64_t n_chunks = (n + rb_grad_reduce_chunk() - 1) / rb_grad_reduce_chunk();
  auto span = torch::zeros({n_chunks, D}, grad_out.options());
  rb_grad_reduce_push(grad_out.data_ptr<float>(), gsrc.data_ptr<int32_t>(), gscale.data_ptr<float>(), csr_u.data_ptr<int32_t>(),
                      csr_elem.data_ptr<int32_t>(), start.data_ptr<int32_t>(), n, (int)D, span.data_ptr<float>(), push, (int)max_blocks, cur_stream());
}

void comm_allreduce_slice(const std::vector<int64_t>& bufs, int64_t me, int64_t n_padded, double scale, bool host) {
  if (host) { rbc_comm_allreduce_slice(peers_of(bufs), (int)me, (int)bufs.size(), n_padded, (float)scale); return; }
  rb_comm_allreduce_slice(peers_of(bufs), (int)me, (int)bufs.size(), n_padded, (float)scale, cur_stream());
}

}  // namespace

void init_comm(py::module& m) {
  m.def("sym_alloc", &sym_alloc);
  m.def("sym_open", &sym_open);
  m.def("sym_close", &sym_close);
  m.def("shm_alloc", &shm_alloc);
  m.def("shm_open_peer", &shm_open_peer);
  m.def("shm_close", &shm_close);
  m.def("shm_unlink_name", &shm_unlink_name);
  m.def("comm_signal", &comm_signal, py::arg("flag_pads"), py::arg("channel"), py::arg("me"), py::arg("epoch"), py::arg("host") = false);
  m.def("comm_wait", &comm_wait);
  m.def("comm_wait_timed", [](const Tensor& flags, int64_t channel, int64_t world, int64_t epoch, int64_t spin_limit, Tensor status,
                              Tensor stats) {
    TORCH_CHECK(stats.scalar_type() == torch::kInt64 && stats.numel() >= RB_CH_COUNT * world + RB_CH_COUNT, "stats: int64 [channels * world + channels]");
    if (!flags.is_cuda()) {
      py::gil_scoped_release nogil;
      rbc_comm_wait_timed(flags.data_ptr<int64_t>(), (int)channel, (int)world, epoch, spin_limit, status.data_ptr<int64_t>(),
                          stats.data_ptr<int64_t>());
      return;
    }
    rb_comm_wait_timed(flags.data_ptr<int64_t>(), (int)channel, (int)world, epoch, spin_limit, status.data_ptr<int64_t>(),
                       stats.data_ptr<int64_t>(), cur_stream());
  });
  m.attr("N_CHANNELS") = (int)RB_CH_COUNT;
  m.def("comm_pull_ids", &comm_pull_ids, py::arg("peer_ids"), py::arg("peer_offsets"), py::arg("peer_counts"), py::arg("me"),
        py::arg("ids_in"), py::arg("prefix"), py::arg("n_in"), py::arg("demand"), py::arg("status"));
  m.def("comm_push_emb", &comm_push_emb, py::arg("emb"), py::arg("rows_in"), py::arg("prefix"), py::arg("peer_uemb"), py::arg("me"),
        py::arg("n_in_hint"), py::arg("blocks") = 0);
  m.def("comm_owner_reduce", &comm_owner_reduce);
  m.def("comm_grad_reduce_push", &comm_grad_reduce_push, py::arg("grad_out"), py::arg("gsrc"), py::arg("gscale"), py::arg("csr_u"),
        py::arg("csr_elem"), py::arg("start"), py::arg("D"), py::arg("offsets"), py::arg("meta"), py::arg("peer_gin"), py::arg("cap_rows"),
        py::arg("max_blocks") = 0);
  m.def("comm_allreduce_slice", &comm_allreduce_slice, py::arg("bufs"), py::arg("me"), py::arg("n_padded"), py::arg("scale"),
        py::arg("host") = false);
  m.def("comm_copy", [](int64_t dst, int64_t src, int64_t nbytes, int64_t blocks) {
    rb_comm_copy(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), nbytes, (int)blocks, cur_stream());
  });
  m.attr("MAX_PEERS") = RB_MAX_PEERS;
}
