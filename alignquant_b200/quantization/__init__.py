"""Artifact format, transform metadata and the quantized Linear module."""
