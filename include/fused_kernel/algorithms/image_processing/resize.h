// Same include path as in FusedKernelLibrary: Resize.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_ALGORITHMS_IMAGE_PROCESSING_RESIZE_H
#define FKB_FWD_ALGORITHMS_IMAGE_PROCESSING_RESIZE_H
#include "../../fkb/frontend.h"
#endif
