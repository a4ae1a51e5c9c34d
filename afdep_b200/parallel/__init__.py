"""Transports and process plumbing: control plane, symmetric-heap bring-up, loopback world."""
