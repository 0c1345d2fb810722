"""Hardware profiles (``hardware_configs/*.json``) and the script that measures them
(reference: galvatron/profile_hardware/)."""
