// Same include path as in FusedKernelLibrary: CircularTensor.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_CORE_DATA_CIRCULAR_TENSOR_H
#define FKB_FWD_CORE_DATA_CIRCULAR_TENSOR_H
#include "../../fkb/frontend.h"
#endif
