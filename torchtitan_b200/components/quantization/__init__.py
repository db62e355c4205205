"""Quantised-training converters (float8 and MXFP8)."""

FP8_GROUP_ALIGNMENT_SIZE = 16
MXFP8_GROUP_ALIGNMENT_SIZE = 32
