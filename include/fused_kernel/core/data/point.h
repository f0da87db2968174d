// Same include path as in FusedKernelLibrary: Point.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_CORE_DATA_POINT_H
#define FKB_FWD_CORE_DATA_POINT_H
#include "../../fkb/frontend.h"
#endif
