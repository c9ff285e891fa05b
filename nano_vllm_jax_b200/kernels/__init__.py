"""Kernel-level ABI (one NHD layer slice) over the C library."""
