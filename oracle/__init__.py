"""CPU oracle of the hot path: test infrastructure, never part of the product."""
