"""Host-side runtime mirroring the reference's ``cleave.runtime`` seams."""
