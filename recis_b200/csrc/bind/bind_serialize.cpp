// Native file layer of the sparse checkpoint: streaming safetensors writer / reader.
//
// File format (identical to the reference's TableWriter, csrc/serialize/table_writer.cc:48-105): u64 header length,
// JSON header padded with spaces to a multiple of 8 bytes (always at least one space), raw tensor bytes.
// A block is either a host tensor or a "gather" block: rows of a device-resident slot slab selected by an index tensor,
// which the writer pulls in chunks of RECIS_BLOCK_WRITE_SIZE rows (default 1 Mi, as csrc/serialize/name.cc:136-152)
// through two pinned staging buffers, so the device-to-host copy of chunk i+1 overlaps the file write of chunk i and the
// host never holds a full copy of a table. Several files are written concurrently, one thread each, with the GIL released.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <fcntl.h>
#include <thread>
#include <unistd.h>
#include "../kernels/rb_kernels.h"
#include "../cpu/rb_cpu.h"
#include "../platform/rb_platform.h"

namespace py = pybind11;
using torch::Tensor;

namespace {

int64_t env_rows(const char* name) {
  const char* v = std::getenv(name);
  return v ? std::max<int64_t>(std::atoll(v), 1) : (1 << 20);
}

struct Block {
  int kind;        // 0 host/dense tensor (copied to CPU by the caller), 1 gather rows of a slab
  Tensor tensor;   // kind 0: contiguous CPU tensor; kind 1: slab [cap, D] fp32 or [cap] int64
  Tensor rows;     // kind 1: int32 row indices on the slab's device
};

struct FileJob {
  std::string path;
  std::string header;
  std::vector<Block> blocks;
  std::string error;
};

using rb::platform::Env;
using rb::platform::FileOutputBuffer;
using rb::platform::FileSystem;
using rb::platform::Status;

void check(const Status& s) {
  if (!s.ok()) throw std::runtime_error(s.ToString());
}

void cuda_ok(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + " failed: " + cudaGetErrorString(e));
}

void write_all(FileOutputBuffer* f, const void* p, size_t n, const std::string& path) {
  if (n) check(f->Append(p, n));
}

void write_gather_block(FileOutputBuffer* f, const Block& b, const std::string& path) {
  const int64_t n = b.rows.numel();
  if (n == 0) return;
  const int64_t D = b.tensor.dim() == 2 ? b.tensor.size(1) : 1;
  const int64_t esz = b.tensor.element_size();
  const int64_t chunk = std::min<int64_t>(env_rows("RECIS_BLOCK_WRITE_SIZE"), n);
  if (!b.tensor.is_cuda()) {
    auto idx = b.rows.to(torch::kInt64);
    for (int64_t s = 0; s < n; s += chunk) {
      auto part = b.tensor.index_select(0, idx.narrow(0, s, std::min(chunk, n - s))).contiguous();
      write_all(f, part.data_ptr(), (size_t)part.numel() * esz, path);
    }
    return;
  }
  c10::cuda::CUDAGuard guard(b.tensor.device());
  auto stream = c10::cuda::getStreamFromPool(false, b.tensor.device().index());
  c10::cuda::CUDAStreamGuard sg(stream);
  Tensor stage_dev[2], stage_host[2];
  cudaEvent_t done[2];
  for (int i = 0; i < 2; ++i) {
    stage_dev[i] = torch::empty({chunk, D}, b.tensor.options());
    stage_host[i] = torch::empty({chunk, D}, b.tensor.options().device(torch::kCPU).pinned_memory(true));
    cuda_ok(cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming), "cudaEventCreate");
  }
  auto issue = [&](int64_t s, int slot) {
    const int64_t m = std::min(chunk, n - s);
    // rows are gathered as bytes: any slab type (fp32 / fp16 / bf16 / int8 rows, int64 per-row counters)
    rb_gather_rows(b.tensor.data_ptr(), b.rows.data_ptr<int32_t>() + s, m, nullptr, D * esz, stage_dev[slot].data_ptr(), stream);
    cuda_ok(cudaMemcpyAsync(stage_host[slot].data_ptr(), stage_dev[slot].data_ptr(), (size_t)m * D * esz, cudaMemcpyDeviceToHost, stream),
            "device-to-host copy of a checkpoint chunk");
    cuda_ok(cudaEventRecord(done[slot], stream), "cudaEventRecord");
  };
  int slot = 0;
  issue(0, 0);
  for (int64_t s = 0; s < n; s += chunk, slot ^= 1) {
    if (s + chunk < n) issue(s + chunk, slot ^ 1);
    // a failed copy must fail the save: the staging buffer would otherwise be written as if it held the rows
    cuda_ok(cudaEventSynchronize(done[slot]), "waiting for a checkpoint chunk");
    write_all(f, stage_host[slot].data_ptr(), (size_t)std::min(chunk, n - s) * D * esz, path);
  }
  for (int i = 0; i < 2; ++i) cudaEventDestroy(done[i]);
}

void run_job(FileJob* job) {
  std::shared_ptr<FileSystem> fs;
  std::string tmp;
  try {
    // written under a temporary name and renamed when complete: a failed save never leaves a half-written shard behind
    std::string local;
    check(Env::Default()->GetFileSystemForFile(job->path, &fs, &local));
    tmp = local + ".tmp";
    std::unique_ptr<rb::platform::WritableFile> wf;
    check(fs->NewWritableFile(tmp, &wf));
    FileOutputBuffer out(std::move(wf), 8u << 20);
    FileOutputBuffer* f = &out;
    std::string header = job->header;
    header.append(8 - (header.size() % 8), ' ');
    const uint64_t hlen = header.size();
    write_all(f, &hlen, sizeof(hlen), tmp);
    write_all(f, header.data(), header.size(), tmp);
    for (const auto& b : job->blocks) {
      if (b.kind == 0) write_all(f, b.tensor.data_ptr(), (size_t)b.tensor.numel() * b.tensor.element_size(), tmp);
      else write_gather_block(f, b, tmp);
    }
    check(out.Close());
    check(fs->RenameFile(tmp, local));
  } catch (const std::exception& e) {
    job->error = e.what();
    if (fs && !tmp.empty() && fs->FileExists(tmp)) (void)fs->DeleteFile(tmp);      // best effort: no stray temporary either
  }
}

// files: list of (path, header json, [ (kind, tensor, rows or None) ... ])
void st_write_files(const std::vector<std::tuple<std::string, std::string, std::vector<std::tuple<int, Tensor, c10::optional<Tensor>>>>>& files) {
  std::vector<FileJob> jobs(files.size());
  for (size_t i = 0; i < files.size(); ++i) {
    jobs[i].path = std::get<0>(files[i]);
    jobs[i].header = std::get<1>(files[i]);
    for (const auto& b : std::get<2>(files[i])) {
      Block blk;
      blk.kind = std::get<0>(b);
      blk.tensor = std::get<1>(b);
      if (blk.kind == 0) {
        TORCH_CHECK(!blk.tensor.is_cuda() && blk.tensor.is_contiguous(), "dense blocks must be contiguous CPU tensors");
      } else {
        TORCH_CHECK(std::get<2>(b).has_value(), "gather blocks need row indices");
        blk.rows = std::get<2>(b)->to(torch::kInt32).contiguous();
        TORCH_CHECK(blk.tensor.is_contiguous());
      }
      jobs[i].blocks.push_back(std::move(blk));
    }
  }
  {
    py::gil_scoped_release nogil;
    std::vector<std::thread> threads;
    for (auto& j : jobs) threads.emplace_back(run_job, &j);
    for (auto& t : threads) t.join();
  }
  for (auto& j : jobs) TORCH_CHECK(j.error.empty(), "checkpoint write failed: ", j.error);
}

std::unique_ptr<rb::platform::RandomAccessFile> open_for_read(const std::string& path) {
  std::shared_ptr<FileSystem> fs;
  std::string local;
  Status s = Env::Default()->GetFileSystemForFile(path, &fs, &local);
  TORCH_CHECK(s.ok(), s.ToString());
  std::unique_ptr<rb::platform::RandomAccessFile> f;
  s = fs->NewRandomAccessFile(local, &f);
  TORCH_CHECK(s.ok(), s.ToString());
  return f;
}

// (header json, offset of the first data byte)
std::tuple<std::string, int64_t> st_read_header(const std::string& path) {
  auto f = open_for_read(path);
  uint64_t hlen = 0;
  size_t got = 0;
  Status s = f->Read(0, sizeof(hlen), &hlen, &got);
  TORCH_CHECK(s.ok() && got == sizeof(hlen) && hlen < (1ull << 32), "corrupt safetensors header in ", path);
  std::string header(hlen, '\0');
  s = f->Read(sizeof(hlen), hlen, header.data(), &got);
  TORCH_CHECK(s.ok() && got == hlen, "truncated safetensors header in ", path);
  return {header, (int64_t)(8 + hlen)};
}

// read `out.nbytes()` bytes at `offset` of `path` into the contiguous CPU tensor `out`
void st_read_into(const std::string& path, int64_t offset, Tensor out) {
  TORCH_CHECK(!out.is_cuda() && out.is_contiguous());
  const size_t n = (size_t)out.numel() * out.element_size();
  char* dst = reinterpret_cast<char*>(out.data_ptr());
  auto f = open_for_read(path);
  size_t got = 0;
  Status s;
  {
    py::gil_scoped_release nogil;
    s = f->Read((uint64_t)offset, n, dst, &got);
  }
  TORCH_CHECK(s.ok(), s.ToString());
  TORCH_CHECK(got == n, "truncated tensor data in ", path, ": wanted ", n, " bytes at ", offset, ", got ", got);
}

// ---- thin Python access to the platform layer (path handling of the checkpoint manager, tests)
bool fs_exists(const std::string& path) {
  std::shared_ptr<FileSystem> fs; std::string local;
  Status s = Env::Default()->GetFileSystemForFile(path, &fs, &local);
  TORCH_CHECK(s.ok(), s.ToString());
  return fs->FileExists(local);
}
int64_t fs_file_size(const std::string& path) {
  std::shared_ptr<FileSystem> fs; std::string local; uint64_t size = 0;
  Status s = Env::Default()->GetFileSystemForFile(path, &fs, &local);
  if (s.ok()) s = fs->GetFileSize(local, &size);
  TORCH_CHECK(s.ok(), s.ToString());
  return (int64_t)size;
}
void fs_mkdirs(const std::string& path) {
  std::shared_ptr<FileSystem> fs; std::string local;
  Status s = Env::Default()->GetFileSystemForFile(path, &fs, &local);
  if (s.ok()) s = fs->CreateDirRecursive(local);
  TORCH_CHECK(s.ok(), s.ToString());
}
void fs_rename(const std::string& from, const std::string& to) {
  std::shared_ptr<FileSystem> fs, fs2; std::string a, b;
  Status s = Env::Default()->GetFileSystemForFile(from, &fs, &a);
  if (s.ok()) s = Env::Default()->GetFileSystemForFile(to, &fs2, &b);
  TORCH_CHECK(s.ok(), s.ToString());
  TORCH_CHECK(fs == fs2, "rename across file systems: ", from, " -> ", to);
  s = fs->RenameFile(a, b);
  TORCH_CHECK(s.ok(), s.ToString());
}
void fs_delete(const std::string& path) {
  std::shared_ptr<FileSystem> fs; std::string local;
  Status s = Env::Default()->GetFileSystemForFile(path, &fs, &local);
  if (s.ok()) s = fs->DeleteFile(local);
  TORCH_CHECK(s.ok(), s.ToString());
}
std::vector<std::string> fs_list(const std::string& dir) {
  std::shared_ptr<FileSystem> fs; std::string local; std::vector<std::string> names;
  Status s = Env::Default()->GetFileSystemForFile(dir, &fs, &local);
  if (s.ok()) s = fs->GetChildren(local, &names);
  TORCH_CHECK(s.ok(), s.ToString());
  std::sort(names.begin(), names.end());
  return names;
}
void fs_write_bytes(const std::string& path, const std::string& data) {
  std::shared_ptr<FileSystem> fs; std::string local;
  Status s = Env::Default()->GetFileSystemForFile(path, &fs, &local);
  TORCH_CHECK(s.ok(), s.ToString());
  std::unique_ptr<rb::platform::WritableFile> wf;
  s = fs->NewWritableFile(local + ".tmp", &wf);
  TORCH_CHECK(s.ok(), s.ToString());
  FileOutputBuffer out(std::move(wf), 1u << 16);
  s = out.Append(data.data(), data.size());
  if (s.ok()) s = out.Close();
  if (s.ok()) s = fs->RenameFile(local + ".tmp", local);
  TORCH_CHECK(s.ok(), s.ToString());
}
py::bytes fs_read_bytes(const std::string& path) {
  const int64_t n = fs_file_size(path);
  std::string buf((size_t)n, '\0');
  auto f = open_for_read(path);
  size_t got = 0;
  Status s = f->Read(0, (size_t)n, buf.data(), &got);
  TORCH_CHECK(s.ok() && got == (size_t)n, "short read of ", path);
  return py::bytes(buf);
}

}  // namespace

void init_serialize(py::module& m) {
  m.def("st_write_files", &st_write_files);
  m.def("st_read_header", &st_read_header);
  m.def("st_read_into", &st_read_into);
  m.def("fs_exists", &fs_exists);
  m.def("fs_file_size", &fs_file_size);
  m.def("fs_mkdirs", &fs_mkdirs);
  m.def("fs_rename", &fs_rename);
  m.def("fs_delete", &fs_delete);
  m.def("fs_list", &fs_list);
  m.def("fs_write_bytes", &fs_write_bytes);
  m.def("fs_read_bytes", &fs_read_bytes);
  m.def("fs_join", &rb::platform::JoinPath);
  m.def("fs_dirname", &rb::platform::Dirname);
  m.def("fs_basename", &rb::platform::Basename);
  m.def("fs_parse_uri", [](const std::string& uri) { std::string sc, p; rb::platform::ParseURI(uri, &sc, &p); return std::make_pair(sc, p); });
  m.def("fs_schemes", []() { return Env::Default()->Schemes(); });
}
