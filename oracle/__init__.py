"""CPU oracle for the KV-block save/load path: test infrastructure, never imported by the product."""
