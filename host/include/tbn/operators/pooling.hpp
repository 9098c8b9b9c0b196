// Same include name as the reference; the declarations live in ops.hpp.
#pragma once
#include "ops.hpp"
