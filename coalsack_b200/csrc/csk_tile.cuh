// Tensor-core grouped contraction (the prefill-side kernel): interface.
#pragma once

#include <functional>
#include <string>

#include "csk_common.cuh"

namespace csk {

constexpr int kTileM = 128;  // rows of a tensor-core row tile

struct TileState {
  bool available = false;
  std::string err;
};

inline int tile_init(TileState& st, int device) {
  (void)device;
  st.available = false;
  return CSK_OK;
}
inline void tile_destroy(TileState&) {}

inline int tile_launch(TileState& st, const uint8_t*, size_t, size_t, size_t, size_t, const MatLayout&,
                       const MatLayout&, const __half*, int, __half*, int, float*, int, const int*,
                       const RowTile*, const int*, int, int, int, int, int, cudaStream_t,
                       const std::function<void()>&) {
  st.err = "not built";
  return CSK_ERR_INVALID;
}

}  // namespace csk
