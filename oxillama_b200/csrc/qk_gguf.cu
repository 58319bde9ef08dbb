// GGUF tensor -> device upload: the bytes of a quantised tensor go from the file into
// pinned staging memory and from there to the GPU, where they are re-tiled; no copy of the
// tensor is ever built in pageable host memory.
//
// Stands where the reference's loader hands a layer its weights:
//   GgufFile::parse             crates/oxillama-gguf/src/parser.rs:34-60   header, metadata, tensor infos,
//                                                                          data offset = position aligned up
//   parse_tensor_infos          parser.rs:166-212                          name, n_dims, dims, type id, offset
//   TensorInfo::data_size       tensor_info.rs:47-56                       ceil(n_elements / block) * block_bytes
//   GgufFile::tensor_data       parser.rs:62-76                            data offset + tensor offset
//   load_quant_linear           crates/oxillama-arch/src/llama/model.rs:805-822
//                               shape = dimensions in file order, rows = shape[0]; data.to_vec()
//
// dimensions[0] is read as the row count (out_features) and dimensions[1] as the column count,
// as the reference does and as its fixtures are written (crates/oxillama-gguf/src/test_utils.rs:183-199).
// A row range of such a tensor is a contiguous byte range of the file, so a row shard is read
// with one pread per staging chunk and nothing else of the tensor is touched.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "qk_internal.h"

struct qk_gguf_tensor {
  std::string name;
  uint32_t n_dims;
  uint64_t dims[4];
  uint32_t type;
  uint64_t offset;  // relative to the data section
};

struct qk_gguf {
  int fd = -1;
  uint64_t file_size = 0, data_offset = 0, alignment = 32;
  uint32_t version = 0;
  std::vector<qk_gguf_tensor> tensors;
  std::map<std::string, size_t> by_name;
  std::string err;
};

namespace {

// Sequential reader over the file's head (header, metadata and tensor infos are read into
// memory in growing pieces; tensor data never is).
struct Cursor {
  int fd;
  uint64_t file_size, pos = 0;
  std::vector<uint8_t> buf;
  uint64_t buf_at = 0;
  bool ok = true;
  bool fill(uint64_t need) {  // make [pos, pos + need) available
    if (pos + need > file_size) return ok = false;
    if (pos >= buf_at && pos + need <= buf_at + buf.size()) return true;
    uint64_t want = need > (1u << 20) ? need : (1u << 20);
    if (pos + want > file_size) want = file_size - pos;
    buf.resize(want);
    uint64_t got = 0;
    while (got < want) {
      ssize_t r = pread(fd, buf.data() + got, want - got, (off_t)(pos + got));
      if (r <= 0) return ok = false;
      got += (uint64_t)r;
    }
    buf_at = pos;
    return true;
  }
  template <typename T>
  T get() {
    T v = T();
    if (!fill(sizeof(T))) return v;
    memcpy(&v, buf.data() + (pos - buf_at), sizeof(T));
    pos += sizeof(T);
    return v;
  }
  std::string str(uint32_t version) {  // v3: u64 length, v1/v2: u32 (reader.rs:177-198)
    uint64_t len = version >= 3 ? get<uint64_t>() : get<uint32_t>();
    if (!ok || len > (1u << 26) || !fill(len)) {
      ok = false;
      return std::string();
    }
    std::string s((const char *)buf.data() + (pos - buf_at), (size_t)len);
    pos += len;
    return s;
  }
  void skip(uint64_t n) {
    if (pos + n > file_size) ok = false;
    pos += n;
  }
};

// Walks over one metadata value (parser.rs:116-163); returns its value as u64 where it is
// an unsigned integer (MetadataValue::as_u64, metadata.rs:89-97), else `none`.
uint64_t skip_value(Cursor &c, uint32_t vtype, uint32_t version, bool *is_uint, int depth = 0) {
  *is_uint = false;
  switch (vtype) {
    case 0: *is_uint = true; return c.get<uint8_t>();
    case 1: c.skip(1); return 0;
    case 2: *is_uint = true; return c.get<uint16_t>();
    case 3: c.skip(2); return 0;
    case 4: *is_uint = true; return c.get<uint32_t>();
    case 5: case 6: c.skip(4); return 0;
    case 7: c.skip(1); return 0;
    case 8: c.str(version); return 0;
    case 10: *is_uint = true; return c.get<uint64_t>();
    case 11: case 12: c.skip(8); return 0;
    case 9: {
      const uint32_t et = c.get<uint32_t>();
      const uint64_t n = version >= 3 ? c.get<uint64_t>() : c.get<uint32_t>();
      if (et > 12 || depth > 8) {
        c.ok = false;
        return 0;
      }
      static const int fixed[13] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};
      if (fixed[et]) {
        c.skip(n * (uint64_t)fixed[et]);
      } else {
        bool dummy;
        for (uint64_t i = 0; i < n && c.ok; i++) skip_value(c, et, version, &dummy, depth + 1);
      }
      return 0;
    }
    default:
      c.ok = false;
      return 0;
  }
}

size_t block_size_of(uint32_t t) { return qk_block_size((int)t); }

}  // namespace

extern "C" int qk_gguf_open(const char *path, qk_gguf **out) {
  if (!path || !out) return QK_INVALID_ARGUMENT;
  *out = nullptr;
  qk_gguf *g = new qk_gguf();
  *out = g;  // returned even on failure, so that qk_gguf_last_error can say why; close it either way
  g->fd = open(path, O_RDONLY);
  struct stat st;
  if (g->fd < 0 || fstat(g->fd, &st) != 0) {
    g->err = std::string("cannot open ") + path;
    return QK_INVALID_ARGUMENT;
  }
  g->file_size = (uint64_t)st.st_size;
  Cursor c{g->fd, g->file_size};
  const uint32_t magic = c.get<uint32_t>();
  if (!c.ok || magic != 0x46554747u) {  // "GGUF" (types.rs:7)
    g->err = "invalid magic";
    return QK_INVALID_ARGUMENT;
  }
  g->version = c.get<uint32_t>();
  if (!c.ok || g->version < 1 || g->version > 3) {  // header.rs:45-47
    g->err = "unsupported GGUF version " + std::to_string(g->version);
    return QK_INVALID_ARGUMENT;
  }
  // counts: u64 in v3, u32 before (header.rs:64-95)
  const uint64_t n_tensors = g->version >= 3 ? c.get<uint64_t>() : c.get<uint32_t>();
  const uint64_t n_kv = g->version >= 3 ? c.get<uint64_t>() : c.get<uint32_t>();
  if (!c.ok || n_tensors > (1u << 24) || n_kv > (1u << 24)) {
    g->err = "truncated or implausible header";
    return QK_INVALID_ARGUMENT;
  }
  for (uint64_t i = 0; i < n_kv; i++) {
    const std::string key = c.str(g->version);
    const uint32_t vtype = c.get<uint32_t>();
    bool is_uint = false;
    const uint64_t v = skip_value(c, vtype, g->version, &is_uint);
    if (!c.ok) {
      g->err = "truncated or malformed metadata at key " + std::to_string(i);
      return QK_INVALID_ARGUMENT;
    }
    if (key == "general.alignment" && is_uint) g->alignment = v;  // parser.rs:42-45
  }
  g->tensors.reserve((size_t)n_tensors);
  for (uint64_t i = 0; i < n_tensors; i++) {
    qk_gguf_tensor t;
    t.name = c.str(g->version);
    t.n_dims = c.get<uint32_t>();
    if (!c.ok || t.n_dims > 4) {
      g->err = "tensor " + std::to_string(i) + ": truncated or more than 4 dimensions";
      return QK_INVALID_ARGUMENT;
    }
    for (int d = 0; d < 4; d++) t.dims[d] = 1;
    for (uint32_t d = 0; d < t.n_dims; d++) t.dims[d] = g->version >= 3 ? c.get<uint64_t>() : c.get<uint32_t>();
    t.type = c.get<uint32_t>();
    t.offset = g->version >= 2 ? c.get<uint64_t>() : c.get<uint32_t>();
    if (!c.ok) {
      g->err = "tensor " + std::to_string(i) + ": truncated";
      return QK_INVALID_ARGUMENT;
    }
    g->by_name[t.name] = g->tensors.size();
    g->tensors.push_back(t);
  }
  const uint64_t a = g->alignment;
  g->data_offset = a ? (c.pos + a - 1) / a * a : c.pos;  // parser.rs:214-225
  return QK_OK;
}

extern "C" int qk_gguf_close(qk_gguf *g) {
  if (!g) return QK_INVALID_ARGUMENT;
  if (g->fd >= 0) close(g->fd);
  delete g;
  return QK_OK;
}

extern "C" int qk_gguf_last_error(const qk_gguf *g, char *buf, size_t len) {
  if (!g || !buf || !len) return QK_INVALID_ARGUMENT;
  snprintf(buf, len, "%s", g->err.c_str());
  return QK_OK;
}

extern "C" int qk_gguf_tensor_count(const qk_gguf *g, size_t *n) {
  if (!g || !n) return QK_INVALID_ARGUMENT;
  *n = g->tensors.size();
  return QK_OK;
}

extern "C" int qk_gguf_tensor_name(const qk_gguf *g, size_t index, char *buf, size_t len) {
  if (!g || !buf || !len || index >= g->tensors.size()) return QK_INVALID_ARGUMENT;
  snprintf(buf, len, "%s", g->tensors[index].name.c_str());
  return QK_OK;
}

// nbytes: TensorInfo::data_size for the five formats this library serves, 0 for other types
// (their block geometry is not known here).  file_offset is absolute.
extern "C" int qk_gguf_tensor_info(const qk_gguf *g, const char *name, int *type, size_t *n_dims, uint64_t dims[4],
                                   uint64_t *file_offset, uint64_t *nbytes) {
  if (!g || !name) return QK_INVALID_ARGUMENT;
  auto it = g->by_name.find(name);
  if (it == g->by_name.end()) return QK_INVALID_ARGUMENT;
  const qk_gguf_tensor &t = g->tensors[it->second];
  if (type) *type = (int)t.type;
  if (n_dims) *n_dims = t.n_dims;
  if (dims)
    for (int d = 0; d < 4; d++) dims[d] = t.dims[d];
  if (file_offset) *file_offset = g->data_offset + t.offset;
  if (nbytes) {
    const size_t bs = block_size_of(t.type), bb = qk_block_bytes((int)t.type);
    uint64_t n = t.n_dims ? 1 : 0;
    for (uint32_t d = 0; d < t.n_dims; d++) n *= t.dims[d];
    *nbytes = bs ? (n + bs - 1) / bs * bb : 0;
  }
  return QK_OK;
}

// Rows [row_begin, row_end) of a 2-D tensor (rows = dimensions[0], columns = dimensions[1];
// a 1-D tensor has n_elements / rows = 1 column, as QuantTensor reads shapes,
// reference/q4_k.rs:110-115), read from the file through two pinned staging buffers (the
// read of piece i + 1 overlaps the copy of piece i) and re-tiled on the device.
extern "C" int qk_weights_upload_gguf(qk_ctx *c, const qk_gguf *g, const char *name, size_t row_begin, size_t row_end,
                                      qk_weights **out) {
  if (!c || !g || !name || !out) return QK_INVALID_ARGUMENT;
  *out = nullptr;
  auto it = g->by_name.find(name);
  if (it == g->by_name.end()) {
    c->err = std::string("no tensor named ") + name;
    return QK_INVALID_ARGUMENT;
  }
  const qk_gguf_tensor &t = g->tensors[it->second];
  const int type = (int)t.type;
  const size_t bs = qk_block_size(type), bb = qk_block_bytes(type);
  if (!bs) {
    c->err = "tensor type id " + std::to_string(t.type) + " is not served by this backend";
    return QK_UNSUPPORTED_TYPE;
  }
  if (t.n_dims < 1 || t.n_dims > 2) return QK_DIMENSION_MISMATCH;
  const uint64_t n_rows = t.dims[0], n_cols = t.n_dims == 2 ? t.dims[1] : 1;
  if (row_begin > row_end || row_end > n_rows || n_rows >= (1ull << 31) || n_cols >= (1ull << 31))
    return QK_INVALID_ARGUMENT;
  const uint64_t row_bytes = (n_cols + bs - 1) / bs * bb;
  const uint64_t rows = row_end - row_begin, nbytes = rows * row_bytes;
  const uint64_t at = g->data_offset + t.offset + row_begin * row_bytes;
  if (at + nbytes > g->file_size) {
    c->err = "tensor data reaches past the end of the file";
    return QK_BUFFER_TOO_SMALL;  // GgufError::UnexpectedEof (parser.rs:71-73)
  }
  std::lock_guard<std::mutex> lk(c->mu);
  if (cudaSetDevice(c->device) != cudaSuccess) return QK_CUDA_ERROR;
  qk_weights *h = new qk_weights();
  h->device = c->device, h->dev = nullptr;
  qk_make_layout(type, rows, n_cols, &h->L);
  h->algo_bytes = nbytes;
  const size_t tiled = h->L.total_bytes ? h->L.total_bytes : 16;
  uint8_t *raw = nullptr, *stage[2] = {nullptr, nullptr};
  cudaEvent_t done[2] = {nullptr, nullptr};
  const size_t piece = (size_t)32 << 20;
  cudaError_t e = cudaMalloc(&h->dev, tiled);
  int st = QK_OK;
  do {
    if (e != cudaSuccess) break;
    if ((e = cudaMemsetAsync(h->dev, 0, tiled, c->stream)) != cudaSuccess) break;
    if (nbytes == 0) break;
    if ((e = cudaMalloc(&raw, nbytes)) != cudaSuccess) break;
    for (int i = 0; i < 2 && e == cudaSuccess; i++) {
      e = cudaHostAlloc((void **)&stage[i], piece < nbytes ? piece : nbytes, cudaHostAllocDefault);
      if (e == cudaSuccess) e = cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming);
    }
    if (e != cudaSuccess) break;
    int k = 0;
    for (uint64_t off = 0; off < nbytes && e == cudaSuccess; off += piece, k ^= 1) {
      const size_t n = (size_t)(nbytes - off < piece ? nbytes - off : piece);
      if (off >= 2 * piece) e = cudaEventSynchronize(done[k]);  // the copy that last used this buffer
      size_t got = 0;
      while (got < n && e == cudaSuccess) {
        ssize_t r = pread(g->fd, stage[k] + got, n - got, (off_t)(at + off + got));
        if (r <= 0) {
          c->err = "read error in the tensor data";
          st = QK_BUFFER_TOO_SMALL;
          break;
        }
        got += (size_t)r;
      }
      if (st != QK_OK) break;
      if (e == cudaSuccess) e = cudaMemcpyAsync(raw + off, stage[k], n, cudaMemcpyHostToDevice, c->stream);
      if (e == cudaSuccess) e = cudaEventRecord(done[k], c->stream);
    }
    if (st != QK_OK || e != cudaSuccess) break;
    e = qk_launch_repack(h->L, raw, h->dev, c->stream);
  } while (0);
  cudaError_t e2 = cudaStreamSynchronize(c->stream);
  if (e == cudaSuccess) e = e2;
  for (int i = 0; i < 2; i++) {
    if (stage[i]) cudaFreeHost(stage[i]);
    if (done[i]) cudaEventDestroy(done[i]);
  }
  if (raw) cudaFree(raw);
  if (e != cudaSuccess || st != QK_OK) {
    if (e != cudaSuccess) {
      c->err = std::string("GGUF tensor upload: ") + cudaGetErrorString(e);
      st = QK_CUDA_ERROR;
    }
    if (h->dev) cudaFree(h->dev);
    delete h;
    return st;
  }
  *out = h;
  return QK_OK;
}
