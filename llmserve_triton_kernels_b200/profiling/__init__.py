"""Profiling aids that are not on the serving path: a timeline of the decode step's kernels from stamps that
the kernels of a profiling build take themselves."""
