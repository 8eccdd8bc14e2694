"""CPU checker for the selective-scan path.  Test infrastructure, not part of the product."""
