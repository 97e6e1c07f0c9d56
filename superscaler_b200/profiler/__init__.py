"""profiler subpackage."""
