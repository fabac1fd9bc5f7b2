#include "rb_platform.h"

#include <dirent.h>
#include <errno.h>
#include <fcntl.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

namespace rb {
namespace platform {

namespace {
Status Errno(const std::string& what, const std::string& path) { return Status::Error(errno ? errno : -1, what + " " + path + ": " + strerror(errno)); }
}  // namespace

std::string JoinPath(const std::string& a, const std::string& b) {
  if (a.empty()) return b;
  if (b.empty()) return a;
  const bool sa = a.back() == '/', sb = b.front() == '/';
  if (sa && sb) return a + b.substr(1);
  if (sa || sb) return a + b;
  return a + "/" + b;
}

std::string Dirname(const std::string& path) {
  const size_t p = path.find_last_of('/');
  if (p == std::string::npos) return "";
  if (p == 0) return "/";
  return path.substr(0, p);
}

std::string Basename(const std::string& path) {
  const size_t p = path.find_last_of('/');
  return p == std::string::npos ? path : path.substr(p + 1);
}

void ParseURI(const std::string& uri, std::string* scheme, std::string* path) {
  const size_t p = uri.find("://");
  bool is_scheme = p != std::string::npos && p > 0;
  for (size_t i = 0; is_scheme && i < p; ++i) {
    const char c = uri[i];
    is_scheme = (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || (c >= '0' && c <= '9') || c == '+' || c == '-' || c == '.';
  }
  if (!is_scheme) { scheme->clear(); *path = uri; return; }
  *scheme = uri.substr(0, p);
  *path = uri.substr(p + 3);
}

// ---------------------------------------------------------------------------------------------- POSIX back end
namespace {

class PosixWritableFile : public WritableFile {
 public:
  PosixWritableFile(std::string path, int fd) : path_(std::move(path)), fd_(fd) {}
  ~PosixWritableFile() override { if (fd_ >= 0) ::close(fd_); }
  Status Append(const void* data, size_t n) override {
    const char* p = static_cast<const char*>(data);
    while (n > 0) {
      const ssize_t w = ::write(fd_, p, n);
      if (w < 0) { if (errno == EINTR) continue; return Errno("write to", path_); }
      p += w; n -= (size_t)w;
    }
    return Status::OK();
  }
  Status Flush() override { return Status::OK(); }
  Status Sync() override { return ::fsync(fd_) == 0 ? Status::OK() : Errno("fsync of", path_); }
  Status Close() override {
    if (fd_ < 0) return Status::OK();
    const int r = ::close(fd_);
    fd_ = -1;
    return r == 0 ? Status::OK() : Errno("close of", path_);
  }

 private:
  std::string path_;
  int fd_;
};

class PosixRandomAccessFile : public RandomAccessFile {
 public:
  PosixRandomAccessFile(std::string path, int fd) : path_(std::move(path)), fd_(fd) {}
  ~PosixRandomAccessFile() override { if (fd_ >= 0) ::close(fd_); }
  Status Read(uint64_t offset, size_t n, void* dst, size_t* got) const override {
    char* p = static_cast<char*>(dst);
    size_t done = 0;
    while (done < n) {
      const ssize_t r = ::pread(fd_, p + done, n - done, (off_t)(offset + done));
      if (r < 0) { if (errno == EINTR) continue; *got = done; return Errno("read of", path_); }
      if (r == 0) break;
      done += (size_t)r;
    }
    *got = done;
    return Status::OK();
  }

 private:
  std::string path_;
  int fd_;
};

class PosixFileSystem : public FileSystem {
 public:
  Status NewWritableFile(const std::string& path, std::unique_ptr<WritableFile>* out) override {
    const int fd = ::open(path.c_str(), O_WRONLY | O_CREAT | O_TRUNC | O_CLOEXEC, 0644);
    if (fd < 0) return Errno("cannot create", path);
    out->reset(new PosixWritableFile(path, fd));
    return Status::OK();
  }
  Status NewRandomAccessFile(const std::string& path, std::unique_ptr<RandomAccessFile>* out) override {
    const int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
    if (fd < 0) return Errno("cannot open", path);
    out->reset(new PosixRandomAccessFile(path, fd));
    return Status::OK();
  }
  bool FileExists(const std::string& path) override { return ::access(path.c_str(), F_OK) == 0; }
  Status GetFileSize(const std::string& path, uint64_t* size) override {
    struct stat st;
    if (::stat(path.c_str(), &st) != 0) return Errno("stat of", path);
    *size = (uint64_t)st.st_size;
    return Status::OK();
  }
  Status CreateDirRecursive(const std::string& path) override {
    if (path.empty() || path == "/") return Status::OK();
    struct stat st;
    if (::stat(path.c_str(), &st) == 0) return S_ISDIR(st.st_mode) ? Status::OK() : Status::Error(ENOTDIR, path + " exists and is not a directory");
    Status s = CreateDirRecursive(Dirname(path));
    if (!s.ok()) return s;
    if (::mkdir(path.c_str(), 0755) != 0 && errno != EEXIST) return Errno("mkdir of", path);
    return Status::OK();
  }
  Status DeleteFile(const std::string& path) override { return ::unlink(path.c_str()) == 0 ? Status::OK() : Errno("unlink of", path); }
  Status RenameFile(const std::string& from, const std::string& to) override {
    return ::rename(from.c_str(), to.c_str()) == 0 ? Status::OK() : Errno("rename of", from + " -> " + to);
  }
  Status GetChildren(const std::string& dir, std::vector<std::string>* names) override {
    DIR* d = ::opendir(dir.c_str());
    if (!d) return Errno("opendir of", dir);
    names->clear();
    while (struct dirent* e = ::readdir(d)) {
      const std::string n = e->d_name;
      if (n != "." && n != "..") names->push_back(n);
    }
    ::closedir(d);
    return Status::OK();
  }
};

}  // namespace

// ---------------------------------------------------------------------------------------------- Env
Env::Env() {
  Factory posix = [] { return std::make_shared<PosixFileSystem>(); };
  factories_[""] = posix;
  factories_["file"] = posix;
}

Env* Env::Default() {
  static Env* env = new Env();
  return env;
}

Status Env::RegisterFileSystem(const std::string& scheme, Factory factory) {
  std::lock_guard<std::mutex> lk(mu_);
  if (factories_.count(scheme)) return Status::Error(EEXIST, "file system for scheme '" + scheme + "' is already registered");
  factories_[scheme] = std::move(factory);
  return Status::OK();
}

Status Env::GetFileSystemForFile(const std::string& uri, std::shared_ptr<FileSystem>* fs, std::string* local_path) {
  std::string scheme;
  ParseURI(uri, &scheme, local_path);
  std::lock_guard<std::mutex> lk(mu_);
  auto it = instances_.find(scheme);
  if (it == instances_.end()) {
    auto f = factories_.find(scheme);
    if (f == factories_.end()) return Status::Error(ENOTSUP, "no file system registered for scheme '" + scheme + "' (" + uri + ")");
    it = instances_.emplace(scheme, f->second()).first;
  }
  *fs = it->second;
  return Status::OK();
}

std::vector<std::string> Env::Schemes() {
  std::lock_guard<std::mutex> lk(mu_);
  std::vector<std::string> out;
  for (auto& kv : factories_) out.push_back(kv.first);
  return out;
}

// ---------------------------------------------------------------------------------------------- FileOutputBuffer
FileOutputBuffer::FileOutputBuffer(std::unique_ptr<WritableFile> file, size_t buffer_bytes) : file_(std::move(file)), buf_(buffer_bytes) {}

FileOutputBuffer::~FileOutputBuffer() { if (!closed_) Close(); }

Status FileOutputBuffer::FlushBuffer() {
  if (used_ == 0) return Status::OK();
  Status s = file_->Append(buf_.data(), used_);
  used_ = 0;
  return s;
}

Status FileOutputBuffer::Append(const void* data, size_t n) {
  written_ += n;
  if (n >= buf_.size()) {                       // large payloads bypass the buffer
    Status s = FlushBuffer();
    return s.ok() ? file_->Append(data, n) : s;
  }
  if (used_ + n > buf_.size()) {
    Status s = FlushBuffer();
    if (!s.ok()) return s;
  }
  memcpy(buf_.data() + used_, data, n);
  used_ += n;
  return Status::OK();
}

Status FileOutputBuffer::Close() {
  if (closed_) return Status::OK();
  closed_ = true;
  Status s = FlushBuffer();
  if (s.ok()) s = file_->Flush();
  if (s.ok()) s = file_->Sync();
  Status c = file_->Close();
  return s.ok() ? c : s;
}

}  // namespace platform
}  // namespace rb
