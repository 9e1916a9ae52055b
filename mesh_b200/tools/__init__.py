"""Command-line tools: launcher/watchdog (meshrun), status (meshctl), profiling drivers."""
