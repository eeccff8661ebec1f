"""CPU oracle for ``frisk.gemm``: test infrastructure only, never imported by frisk_b200/."""
