// placeholder until the tcgen05 kernel lands
#include "common.cuh"
namespace cb2 {
bool decayed_tc_supported(int, int, int, int, int, int, int) { return false; }
int decayed_tc_run(const void*, const void*, const void*, void*, const float*, int, int, int, int,
                   int, int, float, int*, cudaStream_t) { return CB2_BAD_SHAPE; }
}
