"""CPU oracle for the attention path: test infrastructure, never on the product path."""
