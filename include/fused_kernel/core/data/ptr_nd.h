// Same include path as in FusedKernelLibrary: Ptr, Ptr2D, Tensor.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_CORE_DATA_PTR_ND_H
#define FKB_FWD_CORE_DATA_PTR_ND_H
#include "../../fkb/frontend.h"
#endif
