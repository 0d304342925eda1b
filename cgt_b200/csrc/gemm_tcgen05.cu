// placeholder until the tcgen05 kernel lands: reports "shape not supported" so the FMA kernel runs
#include "runtime.h"
namespace cgtb {
int sgemm_tc(int, int, long, long, long, long, const float*, long, long, const float*, long, long, float*, long, long) {
  return -1;
}
}  // namespace cgtb
