// Kept so code written against the reference's include layout compiles unchanged.
#pragma once
#include <vesper/core/tensor.h>
