// Same include path as in FusedKernelLibrary: ColorConversion, ReadYUV, ConvertYUVToRGB.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_ALGORITHMS_IMAGE_PROCESSING_COLOR_CONVERSION_H
#define FKB_FWD_ALGORITHMS_IMAGE_PROCESSING_COLOR_CONVERSION_H
#include "../../fkb/frontend.h"
#endif
