"""Reference arm of the benchmark: runs the unmodified reference package when this image can import it."""
