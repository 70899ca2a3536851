// Epilogue collective types.
// Part of the xefuse_b200 front end: the names live in xefuse/frontend.hpp; this file exists so
// that code including the usual CUTLASS-style path compiles unchanged.
#pragma once
#include "xefuse/frontend.hpp"
