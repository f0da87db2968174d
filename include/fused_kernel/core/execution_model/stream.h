// Same include path as in FusedKernelLibrary: Stream_.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_CORE_EXECUTION_MODEL_STREAM_H
#define FKB_FWD_CORE_EXECUTION_MODEL_STREAM_H
#include "../../fkb/frontend.h"
#endif
