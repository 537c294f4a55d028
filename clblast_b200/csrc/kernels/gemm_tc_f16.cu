#include "launchers.h"
namespace b200 {
cudaError_t launch_tc_f16(const GemmDesc&, cudaStream_t, const char**) { return cudaErrorNotSupported; }
}
