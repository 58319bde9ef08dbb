// Definitions shared by the translation units that implement the C ABI.
#pragma once
#include <map>
#include <mutex>
#include <string>
#include <tuple>

#include "../../include/qk_cuda.h"
#include "qk_kernels.h"

struct qk_weights {
  QkLayout L;
  uint8_t *dev;
  int device;
  size_t algo_bytes;
  uint64_t fp = 0;  // content fingerprint of the host buffer it was uploaded from (host-pointer cache only)
};

struct qk_ctx {
  int device;
  int sm_count;
  cudaStream_t stream;
  // Status word raised by device code (bounded waits that ran out, range checks): one word of
  // pinned host memory that the kernels reach through its device mapping, so the host reads
  // it after a stream synchronise without another copy.
  unsigned *status_dev;                  // device-side address, passed to kernels
  volatile unsigned *status_host = nullptr;  // the same word as the host sees it
  // device scratch of the *_dev entry points (split activations); grown on demand,
  // which synchronises: size it once before capturing into a CUDA graph
  unsigned char *scratch = nullptr;
  size_t scratch_cap = 0;
  std::string err;
  std::mutex mu;
  // scratch for the host-pointer entry points
  void *sa = nullptr, *sb = nullptr;
  size_t sa_cap = 0, sb_cap = 0;
  // weight cache for the host-pointer entry points
  typedef std::tuple<const void *, size_t, int, size_t, size_t, uint64_t> Key;
  std::map<Key, qk_weights *> cache;
  size_t cache_bytes = 0, cache_cap = (size_t)64 << 30;
  bool force_simple = false;
  // scratch of qk_moe_ffn_dev (routing tables and per-expert activations); grown on demand
  void *moe = nullptr;
  size_t moe_cap = 0;
  // scratch of qk_ffn_dev (the hidden activations between the projections); grown on demand
  void *ffn = nullptr;
  size_t ffn_cap = 0;
};

