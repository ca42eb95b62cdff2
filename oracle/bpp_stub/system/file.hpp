/*
 * TEST INFRASTRUCTURE - not part of the shipped library.
 *
 * Stand-in for the one header of the external "bpplib" library that the reference's
 * headers/data.hpp includes (`#include "system/file.hpp"`, data.hpp:7).  bpplib is not part of
 * the reference checkout, and data.hpp needs it only for its R-script export (data.hpp:209-263),
 * which nothing here calls.  With this directory on the include path the reference's own
 * generate_clustered_data and prepare_means (data.hpp:33-81) compile unchanged, so that
 * oracle/ref_data_shim.cpp can expose them and pin the restatement in the command-line harness.
 * The two classes below only have to satisfy the compiler for the unused export templates.
 */
#ifndef BKM_ORACLE_BPP_STUB_FILE_HPP
#define BKM_ORACLE_BPP_STUB_FILE_HPP

#include <string>

namespace bpp {

class File {
public:
	explicit File(const std::string&) {}
	void open() {}
};

class TextWriter {
public:
	TextWriter(File&, const std::string& = "\n", const std::string& = "\t") {}
	template<typename T> void write(const T&) {}
	void writeLine() {}
};

} // namespace bpp

#endif
