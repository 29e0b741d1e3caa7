"""No Pallas here: `scan_mode='pallas'` of the reference cannot be exercised through the shim."""
