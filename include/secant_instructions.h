/*
 * secant_instructions.h - the reference's second header name (program bytecode encoders and
 * decoders, projects/secant/secant_instructions.h), all of which secant_b200.h declares.
 */
#ifndef SECANT_B200_AS_SECANT_INSTRUCTIONS_H
#define SECANT_B200_AS_SECANT_INSTRUCTIONS_H
#include "secant_b200.h"
#endif
