// Same include path as in FusedKernelLibrary: SaturateCast.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_ALGORITHMS_IMAGE_PROCESSING_SATURATE_H
#define FKB_FWD_ALGORITHMS_IMAGE_PROCESSING_SATURATE_H
#include "../../fkb/frontend.h"
#endif
