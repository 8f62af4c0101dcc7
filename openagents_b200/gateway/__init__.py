"""Gateway-side pieces: provider-adapter seam, serve dispatch, admission, router, served-model metadata."""
