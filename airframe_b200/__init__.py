"""airframe_b200: a small model library with generation of its own for one
B200, built from parts: typed configuration and registry, weights by name, a
paged sequence cache, one step function, a generation loop, sampling, and
hand-written sm_100a kernels underneath."""
__version__ = "0.1.0"
