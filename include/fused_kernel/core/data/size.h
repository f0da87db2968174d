// Same include path as in FusedKernelLibrary: Size.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_CORE_DATA_SIZE_H
#define FKB_FWD_CORE_DATA_SIZE_H
#include "../../fkb/frontend.h"
#endif
