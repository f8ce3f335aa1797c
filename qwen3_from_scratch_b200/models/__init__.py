"""Architectures: each module registers a function from its configuration to a ModelSpec."""
