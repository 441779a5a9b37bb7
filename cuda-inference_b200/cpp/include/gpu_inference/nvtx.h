// RAII NVTX range; compiles to nothing unless GIE_HAS_NVTX is defined (drop-in for the reference's nvtx.h).
#pragma once

#ifdef GIE_HAS_NVTX
#include <nvtx3/nvToolsExt.h>
#endif

namespace gie {

class NvtxRange {
 public:
#ifdef GIE_HAS_NVTX
  explicit NvtxRange(const char* label) { nvtxRangePushA(label); }
  ~NvtxRange() { nvtxRangePop(); }
#else
  explicit NvtxRange(const char*) {}
#endif
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

}  // namespace gie
