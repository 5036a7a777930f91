"""CPU oracle for the Heron forward + CE path (test infrastructure only)."""
