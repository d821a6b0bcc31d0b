"""CPU oracle for the kernel parity tests (test infrastructure, not part of the library)."""
