// Stand-in for BOOST_PP_REPEAT_FROM_TO as the reference uses it: always (1, 9, macro, data).
#pragma once
#define BOOST_PP_REPEAT_FROM_TO(first, last, macro, data) \
  macro(0, 1, data) macro(0, 2, data) macro(0, 3, data) macro(0, 4, data) \
  macro(0, 5, data) macro(0, 6, data) macro(0, 7, data) macro(0, 8, data)
