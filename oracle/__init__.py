"""CPU oracle for the LoRA hot path: test infrastructure, never imported by the product."""
