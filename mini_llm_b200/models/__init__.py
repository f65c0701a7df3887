"""Architectures: each module turns its configuration into a model description
and registers itself under the name ``config.json`` gives."""
