"""FP64 CPU checker for the SolveDelta recurrence (test infrastructure only)."""
