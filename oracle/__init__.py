"""CPU oracle of the reference's MoE expert bank: test infrastructure, never a product path."""
