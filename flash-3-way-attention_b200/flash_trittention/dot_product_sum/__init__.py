"""Dot Product Sum trittention."""
