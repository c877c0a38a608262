"""Mixture-of-experts client and server (filled in below)."""
