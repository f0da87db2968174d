// Same include path as in FusedKernelLibrary: PerThreadRead, PerThreadWrite, TensorWrite, TensorSplit.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_ALGORITHMS_BASIC_OPS_MEMORY_OPERATIONS_H
#define FKB_FWD_ALGORITHMS_BASIC_OPS_MEMORY_OPERATIONS_H
#include "../../fkb/frontend.h"
#endif
