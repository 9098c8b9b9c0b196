"""CPU checkers for the tests and the benchmark's CPU-baseline legs.

TEST INFRASTRUCTURE ONLY: nothing in the product package imports this.
"""
