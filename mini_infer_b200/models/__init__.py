"""Architecture assemblies: one file per architecture, each registering itself."""
