// Small platform layer under the native checkpoint code: status values, path helpers, a file-system interface with a registry
// keyed by URI scheme, the POSIX implementation, and a buffered appender.
//
// Same role as the reference's TensorFlow-derived csrc/platform (env.cc:29-81 registry by scheme, posix/posix_filesystem.cc,
// FileOutputBuffer with an 8 MiB buffer used by table_writer.cc:88-104). Only the POSIX back end exists here; the reference's
// optional Pangu back end (fslib) is a service internal to its authors. A path without a scheme, or with "file://", is local.
#pragma once
#include <stdint.h>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace rb {
namespace platform {

class Status {
 public:
  Status() = default;
  static Status OK() { return Status(); }
  static Status Error(int code, std::string msg) { Status s; s.code_ = code; s.msg_ = std::move(msg); return s; }
  bool ok() const { return code_ == 0; }
  int code() const { return code_; }
  const std::string& message() const { return msg_; }
  std::string ToString() const { return ok() ? "OK" : ("error " + std::to_string(code_) + ": " + msg_); }

 private:
  int code_ = 0;
  std::string msg_;
};

// ---- path helpers
std::string JoinPath(const std::string& a, const std::string& b);
std::string Dirname(const std::string& path);
std::string Basename(const std::string& path);
// "scheme://rest" -> (scheme, rest); no scheme -> ("", path)
void ParseURI(const std::string& uri, std::string* scheme, std::string* path);

class WritableFile {
 public:
  virtual ~WritableFile() = default;
  virtual Status Append(const void* data, size_t n) = 0;
  virtual Status Flush() = 0;
  virtual Status Sync() = 0;
  virtual Status Close() = 0;
};

class RandomAccessFile {
 public:
  virtual ~RandomAccessFile() = default;
  // reads up to n bytes at offset; *got receives the count (short only at the end of the file)
  virtual Status Read(uint64_t offset, size_t n, void* dst, size_t* got) const = 0;
};

class FileSystem {
 public:
  virtual ~FileSystem() = default;
  virtual Status NewWritableFile(const std::string& path, std::unique_ptr<WritableFile>* out) = 0;
  virtual Status NewRandomAccessFile(const std::string& path, std::unique_ptr<RandomAccessFile>* out) = 0;
  virtual bool FileExists(const std::string& path) = 0;
  virtual Status GetFileSize(const std::string& path, uint64_t* size) = 0;
  virtual Status CreateDirRecursive(const std::string& path) = 0;
  virtual Status DeleteFile(const std::string& path) = 0;
  virtual Status RenameFile(const std::string& from, const std::string& to) = 0;
  virtual Status GetChildren(const std::string& dir, std::vector<std::string>* names) = 0;
};

class Env {
 public:
  static Env* Default();
  using Factory = std::function<std::shared_ptr<FileSystem>()>;
  Status RegisterFileSystem(const std::string& scheme, Factory factory);
  // resolves the scheme of `uri`; *local_path receives the path as the file system wants it
  Status GetFileSystemForFile(const std::string& uri, std::shared_ptr<FileSystem>* fs, std::string* local_path);
  std::vector<std::string> Schemes();

 private:
  Env();
  std::mutex mu_;
  std::map<std::string, Factory> factories_;
  std::map<std::string, std::shared_ptr<FileSystem>> instances_;
};

// Accumulates appends in a large buffer in front of a WritableFile (the file is owned).
class FileOutputBuffer {
 public:
  explicit FileOutputBuffer(std::unique_ptr<WritableFile> file, size_t buffer_bytes = 8u << 20);
  ~FileOutputBuffer();
  Status Append(const void* data, size_t n);
  Status Close();      // flushes, syncs and closes
  uint64_t bytes_written() const { return written_; }

 private:
  Status FlushBuffer();
  std::unique_ptr<WritableFile> file_;
  std::vector<char> buf_;
  size_t used_ = 0;
  uint64_t written_ = 0;
  bool closed_ = false;
};

}  // namespace platform
}  // namespace rb
