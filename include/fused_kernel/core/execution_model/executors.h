// Same include path as in FusedKernelLibrary: Executor.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_CORE_EXECUTION_MODEL_EXECUTORS_H
#define FKB_FWD_CORE_EXECUTION_MODEL_EXECUTORS_H
#include "../../fkb/frontend.h"
#endif
