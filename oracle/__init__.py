"""CPU oracle for the NVFP4 linear path (test infrastructure; see oracle.py)."""
