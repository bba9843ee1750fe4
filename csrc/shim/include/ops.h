// Reference-compatible entry header: the functionality of the reference's ops.h lives in the
// dg_ops*.h / dg_nn.h headers of this directory (device kernels behind the same names).
#pragma once
#include "dg_nn.h"
