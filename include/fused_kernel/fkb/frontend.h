// The whole front end of the B200 kernels behind FusedKernelLibrary's operator API, in include order.
#pragma once
#include "types.h"
#include "memory.h"
#include "ops.h"
#include "execute.h"
#include "circular_tensor.h"
