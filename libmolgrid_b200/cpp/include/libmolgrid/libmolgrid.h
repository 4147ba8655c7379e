// Single include for the gridding path's C++ interface.
#ifndef LMGB200_LIBMOLGRID_H_
#define LMGB200_LIBMOLGRID_H_
#include "libmolgrid/coordinateset.h"
#include "libmolgrid/grid.h"
#include "libmolgrid/grid_interpolater.h"
#include "libmolgrid/grid_maker.h"
#include "libmolgrid/managed_grid.h"
#include "libmolgrid/quaternion.h"
#include "libmolgrid/transform.h"
#endif
