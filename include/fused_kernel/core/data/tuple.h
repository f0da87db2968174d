// Same include path as in FusedKernelLibrary: buildOperationSequence.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_CORE_DATA_TUPLE_H
#define FKB_FWD_CORE_DATA_TUPLE_H
#include "../../fkb/frontend.h"
#endif
