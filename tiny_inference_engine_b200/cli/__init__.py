"""The command line: `tie generate`, `tie make-random`."""
