// Same include path as in FusedKernelLibrary: Mul, Add, Sub, Div.  The B200 front end lives in fkb/.
#ifndef FKB_FWD_ALGORITHMS_BASIC_OPS_ARITHMETIC_H
#define FKB_FWD_ALGORITHMS_BASIC_OPS_ARITHMETIC_H
#include "../../fkb/frontend.h"
#endif
