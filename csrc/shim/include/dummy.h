// Reference-compatible umbrella header: every op, initialiser, optimizer and module, with the
// reference's global-namespace names, running on the sm_100a kernel library.
// Build a program with:
//   g++ -std=c++20 -I csrc/shim/include prog.cpp -L dummygrad_b200/lib -ldgb200 -Wl,-rpath,<abs path of dummygrad_b200/lib>
#pragma once
#include "dg_nn.h"
