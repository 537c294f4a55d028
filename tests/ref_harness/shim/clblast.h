// The reference's test programs include "clblast.h" (its OpenCL API) unconditionally; under -DCUDA_API they only
// use what the CUDA header declares. This one-line stand-in routes the include to the CUDA header.
#include "clblast_cuda.h"
