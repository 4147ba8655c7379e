// Stand-in for the file the reference's build generates from cmake/config.h.in.
#pragma once
#define VERSION_MAJOR 0
#define VERSION_MINOR 5
#define VERSION_PATCH 3
namespace libmolgrid {
const char* GIT_REVISION = "oracle";
}
