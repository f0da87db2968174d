// Same include path as in FusedKernelLibrary: Cast.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_ALGORITHMS_BASIC_OPS_CAST_H
#define FKB_FWD_ALGORITHMS_BASIC_OPS_CAST_H
#include "../../fkb/frontend.h"
#endif
