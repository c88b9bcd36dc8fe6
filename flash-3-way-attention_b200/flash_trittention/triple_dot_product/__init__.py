"""Triple-dot-product trittention."""
