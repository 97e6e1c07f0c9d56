"""Reference arm of the benchmark (runs the unmodified reference when it can be installed)."""
