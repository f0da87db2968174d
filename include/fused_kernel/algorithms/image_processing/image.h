// Same include path as in FusedKernelLibrary: Image.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_ALGORITHMS_IMAGE_PROCESSING_IMAGE_H
#define FKB_FWD_ALGORITHMS_IMAGE_PROCESSING_IMAGE_H
#include "../../fkb/frontend.h"
#endif
