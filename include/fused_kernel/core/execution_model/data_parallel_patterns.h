// Same include path as in FusedKernelLibrary: TransformDPP, DivergentBatchTransformDPP.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_CORE_EXECUTION_MODEL_DATA_PARALLEL_PATTERNS_H
#define FKB_FWD_CORE_EXECUTION_MODEL_DATA_PARALLEL_PATTERNS_H
#include "../../fkb/frontend.h"
#endif
