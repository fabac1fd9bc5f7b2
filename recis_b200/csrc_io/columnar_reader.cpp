// Native columnar reader: ORC and Parquet files -> training batches, with reader threads, a packer and a prefetch queue.
//
// Pipeline (all C++, the Python caller only pops finished batches):
//   reader threads   decode whole files (Arrow's ORC adapter), up to `threads` files ahead of the packer, in file order;
//   packer thread    cuts each file into batches of `batch_size` rows and packs every configured column into flat tensors:
//                      * variable-length integer columns (int / list<int>)        -> values int64 [nnz] + offsets int32 [rows+1]
//                      * string columns (string / list<string>), hashed at read time with FarmHash64 or MurmurHash64A
//                        (optionally reduced modulo a bucket count)                -> values int64 [nnz] + offsets int32 [rows+1]
//                      * string columns kept as bytes                              -> int8 bytes + row offsets + string offsets
//                      * fixed-length numeric columns                              -> float32 / int64 [rows, 1]
//                    output tensors are optionally pinned; finished batches wait in a bounded queue (`prefetch` deep);
//   next()           pops one batch (the GIL is released while waiting).
// The position after the last batch handed to the caller (file index, row inside the file) is the iterator state: `state()`
// returns it, `restore()` restarts the pipeline from it, so a resumed job continues with the batch it would have seen next.
// Every path may come with a row range [begin, end) of the file (end < 0: to the end of the file): this is how row-addressed
// tables are read (a slice of a table is a list of file segments); rows in the state are always rows of the file.
//
// Same role as the reference's column-io graph (third_party/column-io: ParallelDataset, Packer, PrefetchDataset and
// LocalOrcDataset with read-time hashing, dataset/packer.cc and dataset_impl/local_orc_dataset.cc) with a fixed,
// deterministic order (files in sorted order, rows in file order).
#include <torch/extension.h>

#include <arrow/adapters/orc/adapter.h>
#include <parquet/arrow/reader.h>
#include <arrow/api.h>
#include <arrow/io/file.h>

#include <atomic>
#include <condition_variable>
#include <deque>
#include <limits>
#include <map>
#include <mutex>
#include <thread>

#include "../csrc/common/rb_hash.cuh"

namespace {

struct VarCol { std::string name; int hash_kind; int64_t bucket; bool keep_bytes; };   // hash_kind: -1 none, 0 farm, 1 murmur
struct FixCol { std::string name; double def; };

struct PackedCol {
  int kind;                       // 0 ragged ints (values, offsets); 1 bytes (bytes, row offsets, string offsets); 2 dense
  torch::Tensor a, b, c;
};
struct Batch {
  std::map<std::string, PackedCol> cols;
  int64_t rows = 0, file_idx = 0, next_row = 0;
  bool end = false;
  std::string error;
};

using TablePtr = std::shared_ptr<arrow::Table>;
// What a reader thread hands to the packer: the decoded rows [base, base + table->num_rows()) of a file of n_file rows. An entry
// with a row range decodes only the Parquet row groups / ORC stripes that overlap the range.
struct Decoded { TablePtr table; std::string err; int64_t base = 0; int64_t n_file = 0; };

class ColumnarReader {
 public:
  ColumnarReader(std::vector<std::string> paths, int64_t batch_size, std::vector<VarCol> var, std::vector<FixCol> fix, int threads,
                 int prefetch, bool drop_remainder, bool pin, std::vector<std::pair<int64_t, int64_t>> ranges = {})
      : paths_(std::move(paths)), ranges_(std::move(ranges)), batch_size_(batch_size), var_(std::move(var)), fix_(std::move(fix)),
        threads_(std::max(threads, 1)), prefetch_(std::max(prefetch, 1)), drop_remainder_(drop_remainder), pin_(pin) {
    TORCH_CHECK(batch_size_ > 0, "batch_size must be positive");
    TORCH_CHECK(ranges_.empty() || ranges_.size() == paths_.size(), "one row range per path, or none");
    for (auto& v : var_) names_.push_back(v.name);
    for (auto& f : fix_) names_.push_back(f.name);
    start(0, 0);
  }
  ~ColumnarReader() { stop(); }

  // returns false at the end of the data
  bool next(Batch* out) {
    std::unique_lock<std::mutex> lk(mu_);
    cv_out_.wait(lk, [&] { return !queue_.empty(); });
    if (queue_.front().end) return false;                       // the end marker stays in the queue
    *out = std::move(queue_.front());
    queue_.pop_front();
    cv_in_.notify_all();
    TORCH_CHECK(out->error.empty(), out->error);
    pos_file_ = out->file_idx; pos_row_ = out->next_row;
    return true;
  }
  std::pair<int64_t, int64_t> state() const { return {pos_file_, pos_row_}; }
  void restore(int64_t file_idx, int64_t row) { stop(); start(file_idx, row); }

 private:
  void start(int64_t file_idx, int64_t row) {
    stop_ = false;
    pos_file_ = file_idx; pos_row_ = row;
    next_file_to_read_ = file_idx;
    next_file_to_pack_ = file_idx;
    start_file_ = file_idx;                 // fixed for the life of the threads started below (pos_file_ moves with next())
    first_row_ = row;
    tables_.clear();
    queue_.clear();
    for (int t = 0; t < threads_; ++t) workers_.emplace_back([this] { read_loop(); });
    packer_ = std::thread([this] { pack_loop(); });
  }
  void stop() {
    {
      std::lock_guard<std::mutex> lk(mu_);
      stop_ = true;
    }
    cv_in_.notify_all(); cv_out_.notify_all(); cv_tab_.notify_all();
    for (auto& w : workers_) if (w.joinable()) w.join();
    workers_.clear();
    if (packer_.joinable()) packer_.join();
  }

  // ---- reader threads: claim the next file index, decode it, park the table until the packer takes it
  void read_loop() {
    for (;;) {
      int64_t idx;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_tab_.wait(lk, [&] { return stop_ || next_file_to_read_ - next_file_to_pack_ < threads_ + 1; });
        if (stop_ || next_file_to_read_ >= (int64_t)paths_.size()) return;
        idx = next_file_to_read_++;
      }
      TablePtr table;
      std::string err;
      int64_t base = 0, n_file = 0;
      // rows of the file this entry wants (everything without a range; an end below zero means the end of the file)
      const int64_t want_lo = ranges_.empty() ? 0 : std::max<int64_t>(ranges_[idx].first, 0);
      const int64_t want_hi = ranges_.empty() || ranges_[idx].second < 0 ? std::numeric_limits<int64_t>::max() : ranges_[idx].second;
      auto file = arrow::io::ReadableFile::Open(paths_[idx]);
      const std::string& path = paths_[idx];
      const bool is_parquet = path.size() >= 8 && path.compare(path.size() - 8, 8, ".parquet") == 0;
      if (!file.ok()) err = file.status().ToString();
      else if (is_parquet) {
        // Parquet: the declared columns are selected by name from the file's schema (top-level fields)
        auto reader = parquet::arrow::OpenFile(*file, arrow::default_memory_pool());
        if (!reader.ok()) err = reader.status().ToString();
        else {
          std::shared_ptr<arrow::Schema> schema;
          auto st = (*reader)->GetSchema(&schema);
          std::vector<int> cols;
          if (st.ok()) {
            for (auto& n : names_) {
              const int i = schema->GetFieldIndex(n);
              if (i < 0) { st = arrow::Status::KeyError("no column named ", n); break; }
              cols.push_back(i);
            }
          }
          std::shared_ptr<arrow::Table> t;
          auto md = (*reader)->parquet_reader()->metadata();
          n_file = md->num_rows();
          if (st.ok() && want_hi > want_lo && (want_lo > 0 || want_hi < n_file)) {
            // row groups that overlap [want_lo, want_hi)
            std::vector<int> groups;
            int64_t acc = 0;
            for (int g = 0; g < md->num_row_groups(); ++g) {
              const int64_t n = md->RowGroup(g)->num_rows();
              if (acc + n > want_lo && acc < want_hi) { if (groups.empty()) base = acc; groups.push_back(g); }
              acc += n;
            }
            if (groups.empty()) { base = 0; st = (*reader)->ReadTable(cols, &t); }      // a range past the end: nothing will be packed
            else st = (*reader)->ReadRowGroups(groups, cols, &t);
          } else if (st.ok()) {
            st = (*reader)->ReadTable(cols, &t);
          }
          if (!st.ok()) err = st.ToString();
          else {
            auto c = t->CombineChunks(arrow::default_memory_pool());
            if (!c.ok()) err = c.status().ToString(); else table = *c;
          }
        }
      } else {
        auto reader = arrow::adapters::orc::ORCFileReader::Open(*file, arrow::default_memory_pool());
        if (!reader.ok()) err = reader.status().ToString();
        else {
          n_file = (*reader)->NumberOfRows();
          std::shared_ptr<arrow::Table> t;
          arrow::Status st;
          std::vector<std::shared_ptr<arrow::RecordBatch>> parts;
          if (want_hi > want_lo && (want_lo > 0 || want_hi < n_file)) {
            // stripes that overlap [want_lo, want_hi)
            bool first = true;
            for (int64_t k = 0; k < (*reader)->NumberOfStripes() && st.ok(); ++k) {
              const auto info = (*reader)->GetStripeInformation(k);
              if (info.first_row_id + info.num_rows <= want_lo || info.first_row_id >= want_hi) continue;
              if (first) { base = info.first_row_id; first = false; }
              auto rb = (*reader)->ReadStripe(k, names_);
              if (!rb.ok()) st = rb.status(); else parts.push_back(*rb);
            }
          }
          if (st.ok()) {
            auto r = parts.empty() ? (*reader)->Read(names_) : arrow::Table::FromRecordBatches(parts);
            if (parts.empty()) base = 0;
            if (!r.ok()) st = r.status(); else t = *r;
          }
          if (!st.ok()) err = st.ToString();
          else {
            auto c = t->CombineChunks(arrow::default_memory_pool());
            if (!c.ok()) err = c.status().ToString(); else table = *c;
          }
        }
      }
      {
        std::lock_guard<std::mutex> lk(mu_);
        tables_[idx] = Decoded{table, err.empty() ? "" : ("reading " + paths_[idx] + ": " + err), base, n_file};
      }
      cv_tab_.notify_all();
    }
  }

  // ---- packer thread
  void push(Batch&& b) {
    std::unique_lock<std::mutex> lk(mu_);
    cv_in_.wait(lk, [&] { return stop_ || (int)queue_.size() < prefetch_; });
    if (stop_) return;
    queue_.push_back(std::move(b));
    cv_out_.notify_all();
  }
  void pack_loop() {
    for (int64_t f = next_file_to_pack_; f < (int64_t)paths_.size(); ++f) {
      Decoded item;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_tab_.wait(lk, [&] { return stop_ || tables_.count(f) > 0; });
        if (stop_) return;
        item = tables_[f];
        tables_.erase(f);
        next_file_to_pack_ = f + 1;
      }
      cv_tab_.notify_all();
      if (!item.err.empty()) { Batch b; b.error = item.err; push(std::move(b)); break; }
      // this entry's rows of the file: everything, or the entry's [begin, end); the decoded table starts at row item.base
      const int64_t n_file = item.n_file;
      const int64_t base = item.base;
      const int64_t lo = ranges_.empty() ? 0 : std::min(std::max<int64_t>(ranges_[f].first, 0), n_file);
      const int64_t n = ranges_.empty() || ranges_[f].second < 0 ? n_file : std::min(ranges_[f].second, n_file);
      for (int64_t r0 = (f == start_file_ ? std::max(first_row_, lo) : lo); r0 < n; r0 += batch_size_) {
        const int64_t r1 = std::min(r0 + batch_size_, n);
        if (drop_remainder_ && r1 - r0 < batch_size_) break;
        Batch b;
        b.rows = r1 - r0; b.file_idx = r1 < n ? f : f + 1; b.next_row = r1 < n ? r1 : 0;
        try {
          for (auto& v : var_) b.cols[v.name] = pack_var(*item.table, v, r0 - base, r1 - base);
          for (auto& c : fix_) b.cols[c.name] = pack_fix(*item.table, c, r0 - base, r1 - base);
        } catch (const std::exception& e) {
          b.error = std::string("packing ") + paths_[f] + ": " + e.what();
        }
        const bool failed = !b.error.empty();
        push(std::move(b));
        if (failed || stop_) return;
      }
      first_row_ = 0;
    }
    Batch e; e.end = true;
    push(std::move(e));
  }

  torch::Tensor alloc(std::vector<int64_t> shape, torch::ScalarType t) const {
    return torch::empty(shape, torch::TensorOptions().dtype(t).pinned_memory(pin_));
  }

  static std::shared_ptr<arrow::Array> column(const arrow::Table& t, const std::string& name) {
    auto col = t.GetColumnByName(name);
    if (!col) throw std::runtime_error("no column named " + name);
    if (col->num_chunks() == 0) return nullptr;
    return col->chunk(0);
  }

  template <typename F>
  static void for_each_int(const arrow::Array& arr, int64_t b, int64_t e, F&& f) {      // f(index_in_range, value)
    using arrow::Type;
    auto run = [&](auto* typed) { for (int64_t i = b; i < e; ++i) f(i - b, typed->IsNull(i) ? (int64_t)0 : (int64_t)typed->Value(i)); };
    switch (arr.type_id()) {
      case Type::INT64: run(static_cast<const arrow::Int64Array*>(&arr)); break;
      case Type::INT32: run(static_cast<const arrow::Int32Array*>(&arr)); break;
      case Type::INT16: run(static_cast<const arrow::Int16Array*>(&arr)); break;
      case Type::INT8: run(static_cast<const arrow::Int8Array*>(&arr)); break;
      case Type::UINT64: run(static_cast<const arrow::UInt64Array*>(&arr)); break;
      case Type::UINT32: run(static_cast<const arrow::UInt32Array*>(&arr)); break;
      case Type::BOOL: run(static_cast<const arrow::BooleanArray*>(&arr)); break;
      default: throw std::runtime_error("unsupported integer column type " + arr.type()->ToString());
    }
  }

  PackedCol pack_var(const arrow::Table& t, const VarCol& v, int64_t r0, int64_t r1) const {
    auto arr = column(t, v.name);
    const int64_t rows = r1 - r0;
    PackedCol out;
    auto offs = alloc({rows + 1}, torch::kInt32);
    int32_t* op = offs.data_ptr<int32_t>();
    std::shared_ptr<arrow::Array> flat = arr;
    int64_t f0 = r0, f1 = r1;
    if (arr && arr->type_id() == arrow::Type::LIST) {
      auto* la = static_cast<const arrow::ListArray*>(arr.get());
      f0 = la->value_offset(r0); f1 = la->value_offset(r1);
      for (int64_t i = 0; i <= rows; ++i) op[i] = (int32_t)(la->value_offset(r0 + i) - f0);
      flat = la->values();
    } else {
      for (int64_t i = 0; i <= rows; ++i) op[i] = (int32_t)i;
    }
    const int64_t nnz = f1 - f0;
    const bool is_str = flat && (flat->type_id() == arrow::Type::STRING || flat->type_id() == arrow::Type::BINARY);
    if (is_str) {
      auto* sa = static_cast<const arrow::BinaryArray*>(flat.get());
      if (v.keep_bytes || v.hash_kind < 0) {
        const int64_t b0 = sa->value_offset(f0), b1 = sa->value_offset(f1);
        auto bytes = alloc({b1 - b0}, torch::kInt8);
        if (b1 > b0) std::memcpy(bytes.data_ptr<int8_t>(), sa->raw_data() + b0, (size_t)(b1 - b0));
        auto soff = alloc({nnz + 1}, torch::kInt32);
        int32_t* sp = soff.data_ptr<int32_t>();
        for (int64_t i = 0; i <= nnz; ++i) sp[i] = (int32_t)(sa->value_offset(f0 + i) - b0);
        out.kind = 1; out.a = bytes; out.b = offs; out.c = soff;
        return out;
      }
      auto vals = alloc({nnz}, torch::kInt64);
      int64_t* vp = vals.data_ptr<int64_t>();
      for (int64_t i = 0; i < nnz; ++i) {
        int32_t len = 0;
        const uint8_t* s = sa->GetValue(f0 + i, &len);
        uint64_t h = v.hash_kind == 0 ? rb::hash::farm_fingerprint64(reinterpret_cast<const char*>(s), (size_t)len)
                                      : rb::hash::murmur64a(reinterpret_cast<const char*>(s), (size_t)len, 0);
        if (v.bucket > 0) h %= (uint64_t)v.bucket;
        vp[i] = (int64_t)h;
      }
      out.kind = 0; out.a = vals; out.b = offs;
      return out;
    }
    auto vals = alloc({nnz}, torch::kInt64);
    int64_t* vp = vals.data_ptr<int64_t>();
    if (flat && nnz > 0) {
      for_each_int(*flat, f0, f1, [&](int64_t i, int64_t x) { vp[i] = v.bucket > 0 ? (int64_t)((uint64_t)x % (uint64_t)v.bucket) : x; });
    }
    out.kind = 0; out.a = vals; out.b = offs;
    return out;
  }

  PackedCol pack_fix(const arrow::Table& t, const FixCol& c, int64_t r0, int64_t r1) const {
    auto arr = column(t, c.name);
    const int64_t rows = r1 - r0;
    PackedCol out; out.kind = 2;
    if (arr && (arr->type_id() == arrow::Type::FLOAT || arr->type_id() == arrow::Type::DOUBLE)) {
      out.a = alloc({rows, 1}, torch::kFloat32);
      float* p = out.a.data_ptr<float>();
      if (arr->type_id() == arrow::Type::FLOAT) {
        auto* fa = static_cast<const arrow::FloatArray*>(arr.get());
        for (int64_t i = 0; i < rows; ++i) p[i] = fa->IsNull(r0 + i) ? (float)c.def : fa->Value(r0 + i);
      } else {
        auto* da = static_cast<const arrow::DoubleArray*>(arr.get());
        for (int64_t i = 0; i < rows; ++i) p[i] = da->IsNull(r0 + i) ? (float)c.def : (float)da->Value(r0 + i);
      }
    } else if (arr) {
      out.a = alloc({rows, 1}, torch::kInt64);
      int64_t* p = out.a.data_ptr<int64_t>();
      for_each_int(*arr, r0, r1, [&](int64_t i, int64_t x) { p[i] = x; });
    } else {
      out.a = torch::full({rows, 1}, c.def, torch::kFloat32);
    }
    return out;
  }

  std::vector<std::string> paths_;
  std::vector<std::pair<int64_t, int64_t>> ranges_;       // per path: rows [begin, end) of the file; empty: whole files
  int64_t batch_size_;
  std::vector<VarCol> var_;
  std::vector<FixCol> fix_;
  std::vector<std::string> names_;
  int threads_, prefetch_;
  bool drop_remainder_, pin_;

  std::mutex mu_;
  std::condition_variable cv_in_, cv_out_, cv_tab_;
  std::deque<Batch> queue_;
  std::map<int64_t, Decoded> tables_;
  std::vector<std::thread> workers_;
  std::thread packer_;
  bool stop_ = false;
  int64_t next_file_to_read_ = 0, next_file_to_pack_ = 0, first_row_ = 0, start_file_ = 0;
  int64_t pos_file_ = 0, pos_row_ = 0;
};

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  py::class_<ColumnarReader>(m, "ColumnarReader")
      .def(py::init([](std::vector<std::string> paths, int64_t batch_size, std::vector<std::tuple<std::string, int, int64_t, bool>> var,
                       std::vector<std::tuple<std::string, double>> fix, int threads, int prefetch, bool drop_remainder, bool pin,
                       std::vector<std::pair<int64_t, int64_t>> ranges) {
             std::vector<VarCol> v;
             for (auto& t : var) v.push_back({std::get<0>(t), std::get<1>(t), std::get<2>(t), std::get<3>(t)});
             std::vector<FixCol> f;
             for (auto& t : fix) f.push_back({std::get<0>(t), std::get<1>(t)});
             return new ColumnarReader(std::move(paths), batch_size, std::move(v), std::move(f), threads, prefetch, drop_remainder, pin,
                                       std::move(ranges));
           }),
           py::arg("paths"), py::arg("batch_size"), py::arg("varlen"), py::arg("fixed"), py::arg("threads") = 2, py::arg("prefetch") = 2,
           py::arg("drop_remainder") = false, py::arg("pin") = false, py::arg("ranges") = std::vector<std::pair<int64_t, int64_t>>{})
      .def("next", [](ColumnarReader& r) -> py::object {
             Batch b;
             bool ok;
             {
               py::gil_scoped_release nogil;
               ok = r.next(&b);
             }
             if (!ok) return py::none();
             py::dict d;
             for (auto& kv : b.cols) {
               const PackedCol& c = kv.second;
               if (c.kind == 0) d[py::str(kv.first)] = py::make_tuple(0, c.a, c.b);
               else if (c.kind == 1) d[py::str(kv.first)] = py::make_tuple(1, c.a, c.b, c.c);
               else d[py::str(kv.first)] = py::make_tuple(2, c.a);
             }
             return py::make_tuple(b.rows, d);
           })
      .def("state", &ColumnarReader::state)
      .def("restore", &ColumnarReader::restore);
}
