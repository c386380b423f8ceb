"""Constants shared by host code that must not load the kernel library."""
PAGE = 64   # tokens per cache page; AF_PAGE in csrc/common.cuh
