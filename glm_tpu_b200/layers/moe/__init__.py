"""Mixture of experts: sigmoid top-k router and FP8 routed experts."""
