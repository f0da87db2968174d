// Same include path as in FusedKernelLibrary: BorderReader.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_ALGORITHMS_IMAGE_PROCESSING_BORDER_READER_H
#define FKB_FWD_ALGORITHMS_IMAGE_PROCESSING_BORDER_READER_H
#include "../../fkb/frontend.h"
#endif
