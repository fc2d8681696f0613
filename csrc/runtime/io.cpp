// Checkpoint file primitives: little-endian records with a CRC-32 trailer, byte-compatible with the
// reference formats LTW1 (parameters), LTAD / LTSG / LTRP (optimizer states) and LTDL (loader state)
// (src/serialization/parameters.cpp:9-165, src/serialization/optimizer.cpp:37-393).
//
// A file is: 4-byte magic, a sequence of scalars and tensor records, then the CRC-32 (polynomial
// 0xEDB88320, initial value 0xFFFFFFFF, final xor) of every preceding byte as the last uint32.
// Tensor record: u32 ndims, i64 dim[ndims], u64 numel, f32 data[numel].
// The reader loads the whole file and validates the CRC before it hands out a single value, so a caller
// never mutates its tensors from a corrupt file.  The writer builds the file under a temporary name beside
// the target and renames it over the target when every byte and the CRC are on disk: a process that dies in
// the middle of a save leaves the previous file as it was.
#include "lt_host.h"

#include <unistd.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace {

// Slicing-by-8 CRC-32: eight 256-entry tables, eight input bytes per step (about 2 GB/s per core against 0.4 GB/s for the
// byte-wise loop; a rank's checkpoint shard of an 8B-parameter job is several GB).
struct CrcTable {
  uint32_t v[8][256];
  CrcTable() {
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = i;
      for (int k = 0; k < 8; ++k) c = (c & 1) ? (0xEDB88320u ^ (c >> 1)) : (c >> 1);
      v[0][i] = c;
    }
    for (uint32_t i = 0; i < 256; ++i)
      for (int t = 1; t < 8; ++t) v[t][i] = (v[t - 1][i] >> 8) ^ v[0][v[t - 1][i] & 0xFF];
  }
};

// built once, by whichever thread gets there first (initialisation of a function-local static is thread-safe)
const CrcTable& crc_table() {
  static const CrcTable table;
  return table;
}

uint32_t crc_update(uint32_t crc, const void* data, size_t n) {
  const CrcTable& t = crc_table();
  const uint8_t* p = static_cast<const uint8_t*>(data);
  while (n >= 8) {
    uint32_t lo, hi;
    memcpy(&lo, p, 4);
    memcpy(&hi, p + 4, 4);
    lo ^= crc;                                   // little-endian hosts only (x86-64, aarch64)
    crc = t.v[7][lo & 0xFF] ^ t.v[6][(lo >> 8) & 0xFF] ^ t.v[5][(lo >> 16) & 0xFF] ^ t.v[4][lo >> 24] ^
          t.v[3][hi & 0xFF] ^ t.v[2][(hi >> 8) & 0xFF] ^ t.v[1][(hi >> 16) & 0xFF] ^ t.v[0][hi >> 24];
    p += 8;
    n -= 8;
  }
  for (size_t i = 0; i < n; ++i) crc = t.v[0][(crc ^ p[i]) & 0xFF] ^ (crc >> 8);
  return crc;
}

struct Writer {
  FILE* f = nullptr;
  std::string path, tmp;
  uint32_t crc = 0xFFFFFFFFu;
  bool failed = false;
  void put(const void* d, size_t n) {
    if (failed) return;
    if (n && fwrite(d, 1, n, f) != n) failed = true;
    crc = crc_update(crc, d, n);
  }
};

struct Reader {
  std::vector<uint8_t> buf;
  size_t pos = 0;
  size_t end = 0;  // payload end (before the CRC)
  bool get(void* d, size_t n) {
    if (pos + n > end) return false;
    memcpy(d, buf.data() + pos, n);
    pos += n;
    return true;
  }
};

}  // namespace

extern "C" {

uint32_t lt_crc32(const void* data, uint64_t n) { return crc_update(0xFFFFFFFFu, data, n) ^ 0xFFFFFFFFu; }

void* lt_ckpt_writer_open(const char* path, const char* magic4) {
  const std::string tmp = std::string(path) + ".tmp." + std::to_string(static_cast<long>(getpid()));
  FILE* f = fopen(tmp.c_str(), "wb");
  if (!f) return nullptr;
  Writer* w = new Writer();
  w->f = f;
  w->path = path;
  w->tmp = tmp;
  w->put(magic4, 4);
  return w;
}
int lt_ckpt_write_u32(void* h, uint32_t v) { static_cast<Writer*>(h)->put(&v, 4); return 0; }
int lt_ckpt_write_i32(void* h, int32_t v) { static_cast<Writer*>(h)->put(&v, 4); return 0; }
int lt_ckpt_write_u64(void* h, uint64_t v) { static_cast<Writer*>(h)->put(&v, 8); return 0; }
int lt_ckpt_write_u8(void* h, uint8_t v) { static_cast<Writer*>(h)->put(&v, 1); return 0; }
int lt_ckpt_write_bytes(void* h, const void* d, uint64_t n) { static_cast<Writer*>(h)->put(d, n); return 0; }
int lt_ckpt_write_tensor(void* h, int ndims, const int64_t* dims, const float* data, uint64_t numel) {
  Writer* w = static_cast<Writer*>(h);
  uint32_t nd = uint32_t(ndims);
  w->put(&nd, 4);
  w->put(dims, sizeof(int64_t) * ndims);
  w->put(&numel, 8);
  w->put(data, sizeof(float) * numel);
  return w->failed ? -1 : 0;
}
// Appends the CRC, flushes, closes and publishes the file under its final name. Returns 0 on success, -1 on any
// write failure (disk full...), in which case the target is untouched and the temporary file is removed.
int lt_ckpt_writer_close(void* h) {
  Writer* w = static_cast<Writer*>(h);
  const uint32_t final_crc = w->crc ^ 0xFFFFFFFFu;
  int rc = 0;
  if (!w->failed && fwrite(&final_crc, 1, 4, w->f) != 4) rc = -1;
  if (fflush(w->f) != 0) rc = -1;
  if (rc == 0 && fsync(fileno(w->f)) != 0) rc = -1;
  if (fclose(w->f) != 0) rc = -1;
  if (w->failed) rc = -1;
  if (rc == 0 && rename(w->tmp.c_str(), w->path.c_str()) != 0) rc = -1;
  if (rc != 0) remove(w->tmp.c_str());
  delete w;
  return rc;
}

// err: 0 ok, 1 cannot open, 2 too short, 3 CRC mismatch.
void* lt_ckpt_reader_open(const char* path, char* magic_out4, int* err) {
  *err = 0;
  FILE* f = fopen(path, "rb");
  if (!f) { *err = 1; return nullptr; }
  Reader* r = new Reader();
  fseek(f, 0, SEEK_END);
  long sz = ftell(f);
  fseek(f, 0, SEEK_SET);
  if (sz < 8) { fclose(f); delete r; *err = 2; return nullptr; }
  r->buf.resize(size_t(sz));
  if (fread(r->buf.data(), 1, size_t(sz), f) != size_t(sz)) { fclose(f); delete r; *err = 2; return nullptr; }
  fclose(f);
  r->end = size_t(sz) - 4;
  uint32_t stored;
  memcpy(&stored, r->buf.data() + r->end, 4);
  const uint32_t calc = crc_update(0xFFFFFFFFu, r->buf.data(), r->end) ^ 0xFFFFFFFFu;
  if (stored != calc) { delete r; *err = 3; return nullptr; }
  memcpy(magic_out4, r->buf.data(), 4);
  r->pos = 4;
  return r;
}
int lt_ckpt_read_u32(void* h, uint32_t* v) { return static_cast<Reader*>(h)->get(v, 4) ? 0 : -1; }
int lt_ckpt_read_i32(void* h, int32_t* v) { return static_cast<Reader*>(h)->get(v, 4) ? 0 : -1; }
int lt_ckpt_read_u64(void* h, uint64_t* v) { return static_cast<Reader*>(h)->get(v, 8) ? 0 : -1; }
int lt_ckpt_read_u8(void* h, uint8_t* v) { return static_cast<Reader*>(h)->get(v, 1) ? 0 : -1; }
int lt_ckpt_read_bytes(void* h, void* d, uint64_t n) { return static_cast<Reader*>(h)->get(d, n) ? 0 : -1; }
uint64_t lt_ckpt_remaining(void* h) { Reader* r = static_cast<Reader*>(h); return r->end - r->pos; }
// Reads the header of the next tensor record without its data (dims: room for 16 entries).
int lt_ckpt_read_tensor_header(void* h, int* ndims, int64_t* dims, uint64_t* numel) {
  Reader* r = static_cast<Reader*>(h);
  uint32_t nd;
  if (!r->get(&nd, 4) || nd > 16) return -1;
  if (!r->get(dims, sizeof(int64_t) * nd)) return -1;
  if (!r->get(numel, 8)) return -1;
  uint64_t prod = 1;
  for (uint32_t i = 0; i < nd; ++i) {
    if (dims[i] < 0) return -1;
    prod *= uint64_t(dims[i]);
  }
  if (prod != *numel) return -2;
  if (r->pos + *numel * sizeof(float) > r->end) return -1;
  *ndims = int(nd);
  return 0;
}
int lt_ckpt_read_tensor_data(void* h, float* out, uint64_t numel) {
  return static_cast<Reader*>(h)->get(out, numel * sizeof(float)) ? 0 : -1;
}
void lt_ckpt_reader_close(void* h) { delete static_cast<Reader*>(h); }

}  // extern "C"
