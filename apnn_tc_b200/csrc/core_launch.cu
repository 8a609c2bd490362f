// Dispatch of the warp-level plane contraction core over the instantiated width pairs.
#include "core_launch.h"

namespace apnn {

template <int AB, int BB>
cudaError_t launch_pair(int kind, const CoreParams& p, cudaStream_t s, int tile_class);

#define APNN_PAIRS(X) X(1, 1) X(1, 2) X(1, 3) X(1, 4) X(2, 1) X(3, 1) X(4, 1) X(2, 2)
#define APNN_DECL(AB, BB) extern template cudaError_t launch_pair<AB, BB>(int, const CoreParams&, cudaStream_t, int);
APNN_PAIRS(APNN_DECL)
#undef APNN_DECL

bool core_supports(int abits, int bbits) {
#define APNN_TEST(AB, BB) if (abits == AB && bbits == BB) return true;
  APNN_PAIRS(APNN_TEST)
#undef APNN_TEST
  return false;
}

int core_pick_tile(const CoreParams& p, int sm_count) {
  long long big_tiles = (((long long)p.M + 127) / 128) * (((long long)p.N + 127) / 128);
  return big_tiles * 2 >= sm_count ? TILE_BIG : TILE_SMALL;
}

cudaError_t launch_core(int kind, int abits, int bbits, const CoreParams& p, cudaStream_t s, int tile_class) {
#define APNN_CASE(AB, BB) if (abits == AB && bbits == BB) return launch_pair<AB, BB>(kind, p, s, tile_class);
  APNN_PAIRS(APNN_CASE)
#undef APNN_CASE
  return cudaErrorInvalidValue;
}

}  // namespace apnn
