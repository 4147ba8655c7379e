// Stand-in so the reference's grid.h can be included without Boost; the header is never used there.
#pragma once
