// Same include path as in FusedKernelLibrary: RawPtr, PtrDims.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_CORE_DATA_RAWPTR_H
#define FKB_FWD_CORE_DATA_RAWPTR_H
#include "../../fkb/frontend.h"
#endif
