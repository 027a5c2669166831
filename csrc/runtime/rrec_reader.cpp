// Memory-mapped reader for the `.rrec` record format (C ABI, loaded with ctypes).
//
// File layout (rumus/src/data/record.rs:1-20,84-141):
//   header 64 B : "RREC" | u32 version = 1 | u64 num_records | u64 index_offset | 40 B reserved
//   records     : (input tensor, target tensor), each  u32 ndim | u32 shape[ndim] | u32 dtype
//                 (0 = f32, 1 = f16) | raw little-endian data | zero padding to 4 bytes
//   index       : num_records x (u64 offset, u64 length)
// The reader maps the file once; every accessor validates offsets against the mapping size and
// hands back pointers into the mapping (no copy).
#include <cstdint>
#include <cstring>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace {
struct Rrec {
  const uint8_t* base;
  size_t size;
  uint64_t n;
  uint64_t index_off;
};
uint32_t rd32(const uint8_t* p) { uint32_t v; std::memcpy(&v, p, 4); return v; }
uint64_t rd64(const uint8_t* p) { uint64_t v; std::memcpy(&v, p, 8); return v; }
}  // namespace

extern "C" {

void* rrec_open(const char* path) {
  int fd = ::open(path, O_RDONLY);
  if (fd < 0) return nullptr;
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < 64) { ::close(fd); return nullptr; }
  void* m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (m == MAP_FAILED) return nullptr;
  const uint8_t* b = static_cast<const uint8_t*>(m);
  if (std::memcmp(b, "RREC", 4) != 0 || rd32(b + 4) != 1) { munmap(m, (size_t)st.st_size); return nullptr; }
  Rrec* r = new Rrec{b, (size_t)st.st_size, rd64(b + 8), rd64(b + 16)};
  if (r->index_off + r->n * 16 > r->size) { munmap(m, r->size); delete r; return nullptr; }
  return r;
}

void rrec_close(void* h) {
  Rrec* r = static_cast<Rrec*>(h);
  if (!r) return;
  munmap(const_cast<uint8_t*>(r->base), r->size);
  delete r;
}

long long rrec_len(void* h) { return (long long)static_cast<Rrec*>(h)->n; }

// which: 0 = input tensor, 1 = target tensor of record `idx`.
// Fills ndim, shape (up to 8 dims), dtype tag and a pointer to the raw data; returns the data size
// in bytes or -1 on a malformed record.
long long rrec_tensor(void* h, long long idx, int which, int* ndim, int* shape, int* dtype,
                      const void** data) {
  Rrec* r = static_cast<Rrec*>(h);
  if (idx < 0 || (uint64_t)idx >= r->n) return -1;
  const uint8_t* e = r->base + r->index_off + (uint64_t)idx * 16;
  uint64_t off = rd64(e), len = rd64(e + 8);
  if (off + len > r->size) return -1;
  const uint8_t* p = r->base + off;
  const uint8_t* end = p + len;
  for (int t = 0; t <= which; ++t) {
    if (p + 4 > end) return -1;
    const uint32_t nd = rd32(p);
    if (nd > 8 || p + 8 + 4 * (size_t)nd > end) return -1;
    uint64_t numel = 1;
    for (uint32_t i = 0; i < nd; ++i) numel *= rd32(p + 4 + 4 * i);
    const uint32_t tag = rd32(p + 4 + 4 * nd);
    const uint64_t bytes = numel * (tag == 1 ? 2 : 4);
    const uint8_t* d = p + 8 + 4 * nd;
    if (d + bytes > end) return -1;
    if (t == which) {
      *ndim = (int)nd;
      for (uint32_t i = 0; i < nd; ++i) shape[i] = (int)rd32(p + 4 + 4 * i);
      *dtype = (int)tag;
      *data = d;
      return (long long)bytes;
    }
    p = d + ((bytes + 3) & ~3ull);
  }
  return -1;
}
}
