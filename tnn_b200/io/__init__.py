"""Binary formats: TNNG graph-state checkpoints, raw tensor records, archiver wire messages."""
