/*
 * TEST INFRASTRUCTURE — CPU oracle for the WKV7 hot path (see wkv7_oracle_impl.h).
 * Exports every function twice: suffix _f32 (float) and _f64 (double).
 * Build: gcc -O3 -march=native -fopenmp -shared -fPIC wkv7_oracle.c -o _build/libwkv7_oracle.so -lm
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#define MAXN 256

#define REAL float
#define SUFFIX _f32
#include "wkv7_oracle_impl.h"
#undef REAL
#undef SUFFIX

#define REAL double
#define SUFFIX _f64
#include "wkv7_oracle_impl.h"
#undef REAL
#undef SUFFIX
