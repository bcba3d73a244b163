"""Convolution layers of the hot path (KPConv, MCConv)."""
