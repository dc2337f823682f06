"""Model configurations and the shared command-line plumbing of the benchmark entry points."""
