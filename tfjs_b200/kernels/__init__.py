"""Kernel configs of the 'cuda' backend, one per name in
tfjs-core/src/kernel_names.ts that the inference hot path uses."""
