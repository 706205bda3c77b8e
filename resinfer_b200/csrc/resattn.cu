// placeholder translation unit (filled in below)
