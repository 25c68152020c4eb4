/*
 * secant.h - the reference header's name for this library's C API.
 *
 * A consumer written against the reference (`#include "secant.h"`) compiles against this
 * repository's include directory unchanged: every type, constant, inline helper and entry point
 * the reference header declares for the population-evaluation path is declared by secant_b200.h.
 */
#ifndef SECANT_B200_AS_SECANT_H
#define SECANT_B200_AS_SECANT_H
#include "secant_b200.h"
#endif
