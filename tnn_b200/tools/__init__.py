"""Command-line helpers that sit beside the framework: telemetry sampler and profiler timeline export."""
