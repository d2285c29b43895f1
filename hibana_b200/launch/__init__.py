"""Launcher: settings resolution, rank supervisor, memory guard, preflight checks, control clients."""
