// Read-only memory-mapped file (RAII).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

namespace pocket {

class MappedFile {
 public:
  MappedFile() = default;
  explicit MappedFile(const std::string& path);   // throws std::runtime_error
  ~MappedFile();
  MappedFile(MappedFile&& o) noexcept;
  MappedFile& operator=(MappedFile&& o) noexcept;
  MappedFile(const MappedFile&) = delete;
  MappedFile& operator=(const MappedFile&) = delete;
  const uint8_t* data() const { return data_; }
  size_t size() const { return size_; }
  const std::string& path() const { return path_; }
  void advise_willneed(size_t offset, size_t length) const;

 private:
  void reset();
  const uint8_t* data_ = nullptr;
  size_t size_ = 0;
  std::string path_;
};

}  // namespace pocket
