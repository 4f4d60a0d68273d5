// Status word shared by every kernel: the first failure wins, the host reads it after a sync.
#pragma once

namespace zx {

enum : int {
  ZX_OK = 0,
  ZX_ERR_TIMEOUT = 1,  // a bounded wait ran out
  ZX_ERR_BOUNDS = 2,   // checked mode: an index fell outside its descriptor
  ZX_ERR_ARG = 3,
};

struct Status {
  int code;   // ZX_OK or the first error
  int site;   // which wait / check
  int block;  // blockIdx.x that reported
  int info;   // site-specific
};

}  // namespace zx
