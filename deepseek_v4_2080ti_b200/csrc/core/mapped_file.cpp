#include "mapped_file.hpp"

#include <stdexcept>
#include <utility>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace pocket {

MappedFile::MappedFile(const std::string& path) : path_(path) {
  int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
  if (fd < 0) throw std::runtime_error("cannot open " + path);
  struct stat st;
  if (::fstat(fd, &st) != 0) { ::close(fd); throw std::runtime_error("cannot stat " + path); }
  size_ = static_cast<size_t>(st.st_size);
  if (size_ > 0) {
    void* p = ::mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd, 0);
    if (p == MAP_FAILED) { ::close(fd); throw std::runtime_error("cannot mmap " + path); }
    data_ = static_cast<const uint8_t*>(p);
  }
  ::close(fd);
}

void MappedFile::reset() {
  if (data_) ::munmap(const_cast<uint8_t*>(data_), size_);
  data_ = nullptr;
  size_ = 0;
}

MappedFile::~MappedFile() { reset(); }

MappedFile::MappedFile(MappedFile&& o) noexcept : data_(o.data_), size_(o.size_), path_(std::move(o.path_)) {
  o.data_ = nullptr;
  o.size_ = 0;
}

MappedFile& MappedFile::operator=(MappedFile&& o) noexcept {
  if (this != &o) {
    reset();
    data_ = o.data_;
    size_ = o.size_;
    path_ = std::move(o.path_);
    o.data_ = nullptr;
    o.size_ = 0;
  }
  return *this;
}

void MappedFile::advise_willneed(size_t offset, size_t length) const {
  if (!data_ || offset >= size_) return;
  if (offset + length > size_) length = size_ - offset;
  const size_t page = 4096;
  const size_t lo = offset / page * page;
  ::madvise(const_cast<uint8_t*>(data_) + lo, length + (offset - lo), MADV_WILLNEED);
}

}  // namespace pocket
