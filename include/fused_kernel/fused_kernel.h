// Same include path as in FusedKernelLibrary: the user entry points (fk::executeOperations, Executor).  The B200 front end lives in fkb/.
#ifndef FKB_FWD_FUSED_KERNEL_H
#define FKB_FWD_FUSED_KERNEL_H
#include "fkb/frontend.h"
#endif
