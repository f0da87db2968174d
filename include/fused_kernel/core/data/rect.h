// Same include path as in FusedKernelLibrary: Rect.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_CORE_DATA_RECT_H
#define FKB_FWD_CORE_DATA_RECT_H
#include "../../fkb/frontend.h"
#endif
