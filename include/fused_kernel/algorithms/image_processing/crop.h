// Same include path as in FusedKernelLibrary: Crop.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_ALGORITHMS_IMAGE_PROCESSING_CROP_H
#define FKB_FWD_ALGORITHMS_IMAGE_PROCESSING_CROP_H
#include "../../fkb/frontend.h"
#endif
