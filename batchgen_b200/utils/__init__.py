"""Event log, timers, memfd helpers."""
