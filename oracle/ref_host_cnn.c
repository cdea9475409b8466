/* CNN drivers: filled in below */
