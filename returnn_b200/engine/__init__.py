"""Engine base and legacy batch containers."""
