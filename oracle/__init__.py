"""CPU oracle for the NVFP4 projection path: test infrastructure, never imported by the product package."""
